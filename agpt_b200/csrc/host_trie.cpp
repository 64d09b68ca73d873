// Host side of libagpt_b200: synthetic workloads, radix-trie construction and directory
// I/O, the char-position tree, the depth-first walker plan and the unit partitioner.
//
// The trie builder reproduces the node numbering of the reference's two-stage build
// (src/agpt/streaming_leveled_builder.cr:31-118 then src/agpt/streaming_radix_builder.cr:103-343)
// without materialising per-depth hash groups: suffix start positions are kept bucketed by
// their current trie node and each level refines every bucket with a counting sort on the
// next token, which yields nodes in (parent id, token) order directly.
#include <cuda_runtime.h>

#include <algorithm>
#include <cmath>
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <deque>
#include <map>
#include <numeric>
#include <string>
#include <vector>

#include "../../include/agpt_b200.h"
#include "internal.h"

// --------------------------------------------------------------------------------------
// errors
// --------------------------------------------------------------------------------------
static thread_local char g_err[512] = "";

int agpt_set_error(int code, const char *fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
    return code;
}

extern "C" const char *agpt_b200_last_error(void) { return g_err; }
extern "C" const char *agpt_b200_version(void) { return "agpt_b200 0.1 (sm_100a)"; }

// --------------------------------------------------------------------------------------
// synthetic workloads
// --------------------------------------------------------------------------------------
static inline uint64_t splitmix64(uint64_t x) {
    x += 0x9E3779B97F4A7C15ULL;
    uint64_t z = x;
    z = (z ^ (z >> 30)) * 0xBF58476D1CE4E5B9ULL;
    z = (z ^ (z >> 27)) * 0x94D049BB133111EBULL;
    return z ^ (z >> 31);
}
static inline double u01(uint64_t z) { return (double)(z >> 11) * (1.0 / 9007199254740992.0); }

static int inv_cdf(const std::vector<double> &cdf, double u) {
    int lo = 0, hi = (int)cdf.size() - 1;
    while (lo < hi) {
        int mid = (lo + hi) / 2;
        if (u < cdf[mid]) hi = mid; else lo = mid + 1;
    }
    return lo;
}

static int synth_markov(int64_t n, int vocab, int order, uint64_t seed, int repeat_log2, int32_t *out);

extern "C" int agpt_b200_synth_markov_corpus(int64_t n, int vocab, int order, uint64_t seed, int32_t *out) {
    return synth_markov(n, vocab, order, seed, 0, out);
}

extern "C" int agpt_b200_synth_markov_corpus_repeats(int64_t n, int vocab, int order, uint64_t seed, int repeat_log2,
                                                     int32_t *out) {
    if (repeat_log2 < 1 || repeat_log2 > 40) return agpt_set_error(AGPT_E_ARG, "synth_markov_corpus_repeats: repeat_log2 must be 1..40");
    return synth_markov(n, vocab, order, seed, repeat_log2, out);
}

// repeat_log2 > 0: before each symbol one more draw of the stream decides, with probability 2^-repeat_log2, to copy
// a span of 64 + (draw mod 193) symbols from a uniformly drawn earlier offset instead (long verbatim repeats, as
// natural text has them; a plain low-order Markov source has none, so its count>=2 trie stays shallow).
static int synth_markov(int64_t n, int vocab, int order, uint64_t seed, int repeat_log2, int32_t *out) {
    if (!out || n < 0 || vocab < 2 || order < 1 || order > 8) return agpt_set_error(AGPT_E_ARG, "synth_markov_corpus: bad argument");
    const int M = 6;
    std::vector<double> zipf(vocab), slot(M);
    double tot = 0;
    for (int r = 0; r < vocab; r++) { tot += std::pow((double)(r + 1), -1.1); zipf[r] = tot; }
    for (auto &c : zipf) c /= tot;
    zipf[vocab - 1] = 1.0;
    tot = 0;
    for (int r = 0; r < M; r++) { tot += std::pow((double)(r + 1), -1.1); slot[r] = tot; }
    for (auto &c : slot) c /= tot;
    slot[M - 1] = 1.0;
    uint64_t modulus = 1;
    for (int i = 0; i < order; i++) modulus *= (uint64_t)vocab;
    uint64_t ctx = 0, s = splitmix64(seed);
    for (int64_t i = 0; i < n; i++) {
        if (repeat_log2 > 0 && i > 0) {
            s = splitmix64(s);
            if ((s >> (64 - repeat_log2)) == 0) {
                s = splitmix64(s);
                const int64_t len = 64 + (int64_t)(s % 193);
                s = splitmix64(s);
                const int64_t src = (int64_t)(s % (uint64_t)i);
                int64_t t = 0;
                for (; t < len && i + t < n; t++) {          // the span may run into what it is writing (like an LZ77 match)
                    const int sym = out[src + t];
                    out[i + t] = sym;
                    ctx = (ctx * (uint64_t)vocab + (uint64_t)sym) % modulus;
                }
                i += t - 1;
                continue;
            }
        }
        uint64_t h = splitmix64(seed ^ (ctx * 0x9E3779B97F4A7C15ULL));
        s = splitmix64(s);
        int j = inv_cdf(slot, u01(s));
        int sym = 0;
        for (int d = 0; d <= j; d++) { h = splitmix64(h); sym = inv_cdf(zipf, u01(h)); }
        out[i] = sym;
        ctx = (ctx * (uint64_t)vocab + (uint64_t)sym) % modulus;
    }
    return AGPT_OK;
}

extern "C" int64_t agpt_b200_synth_tree(int64_t max_nodes, int max_depth, int root_children, double p_stop,
                                         int max_children, int64_t level_cap, uint64_t seed, int32_t *parent_out) {
    if (!parent_out || max_nodes <= 0 || max_depth < 1 || root_children < 1 || p_stop <= 0 || p_stop > 1)
        return agpt_set_error(AGPT_E_ARG, "synth_tree: bad argument");
    uint64_t s = splitmix64(seed ^ 0xA5A5A5A5ULL);
    int64_t n = 0, lvl_begin = 0, lvl_end = 0;
    for (int c = 0; c < root_children && n < max_nodes; c++) parent_out[n++] = -1;
    lvl_end = n;
    for (int d = 2; d <= max_depth && n < max_nodes && lvl_end > lvl_begin; d++) {
        int64_t width = 0;
        for (int64_t i = lvl_begin; i < lvl_end && n < max_nodes && width < level_cap; i++) {
            int c = 0;
            for (;;) {
                s = splitmix64(s);
                if (u01(s) < p_stop || c >= max_children) break;
                c++;
            }
            for (int k = 0; k < c && n < max_nodes && width < level_cap; k++) { parent_out[n++] = (int32_t)i; width++; }
        }
        lvl_begin = lvl_end;
        lvl_end = n;
    }
    return n;
}

// RoPE tables in float32 host arithmetic, value duplicated over each (2i, 2i+1) pair.
extern "C" int agpt_b200_rope_table(float *cos_out, float *sin_out, int max_seq, int head_dim, float base) {
    if (!cos_out || !sin_out || max_seq < 1 || head_dim < 2 || head_dim % 2) return agpt_set_error(AGPT_E_ARG, "rope_table: bad argument");
    for (int pos = 0; pos < max_seq; pos++)
        for (int i = 0; i < head_dim / 2; i++) {
            float theta = pos / powf(base, 2.0f * i / head_dim);
            float c = cosf(theta), s = sinf(theta);
            cos_out[pos * head_dim + 2 * i] = cos_out[pos * head_dim + 2 * i + 1] = c;
            sin_out[pos * head_dim + 2 * i] = sin_out[pos * head_dim + 2 * i + 1] = s;
        }
    return AGPT_OK;
}

// --------------------------------------------------------------------------------------
// radix trie
// --------------------------------------------------------------------------------------
namespace {
// Depth-capped suffix trie in level order; children of a node are id-contiguous.
struct Leveled {
    std::vector<int32_t> token, first_child, child_count;
    std::vector<int64_t> cnt_off;
    std::vector<int32_t> cnt_tok, cnt_val;
    int32_t n_levels = 1;
};

void build_leveled(const int32_t *corpus, int64_t n, int max_depth, int vocab, Leveled &L) {
    L.token.assign(1, -1);
    L.first_child.assign(1, -1);
    L.child_count.assign(1, 0);
    L.cnt_off.assign(2, 0);
    // cursors bucketed by node: cur[] holds corpus positions, bucket b covers [boff[b], boff[b+1]) and
    // belongs to node bnode[b] of the previous level
    int64_t n_act = n > 0 ? n - 1 : 0;
    std::vector<int32_t> cur(n_act), nxt(n_act), bnode{0};
    std::vector<int64_t> boff{0, n_act};
    std::iota(cur.begin(), cur.end(), 0);
    std::vector<int64_t> hist(vocab + 1);
    for (int d = 1; d <= max_depth && n_act > 0; d++) {
        std::vector<int32_t> nb_node;
        std::vector<int64_t> nb_off{0};
        int64_t out = 0;
        for (size_t b = 0; b + 1 < boff.size(); b++) {
            int64_t lo = boff[b], hi = boff[b + 1];
            int32_t par = bnode[b];
            std::fill(hist.begin(), hist.end(), 0);
            for (int64_t i = lo; i < hi; i++) hist[corpus[cur[i]] + 1]++;
            // node per non-empty token bucket, in token order
            int32_t first = -1, cnt = 0;
            std::vector<std::pair<int32_t, int32_t>> toks;  // (token, node id)
            for (int t = 0; t < vocab; t++)
                if (hist[t + 1]) {
                    int32_t nid = (int32_t)L.token.size();
                    L.token.push_back(t);
                    L.first_child.push_back(-1);
                    L.child_count.push_back(0);
                    if (first < 0) first = nid;
                    cnt++;
                    toks.emplace_back(t, nid);
                }
            L.first_child[par] = first;
            L.child_count[par] = cnt;
            for (int t = 0; t < vocab; t++) hist[t + 1] += hist[t];
            // stable scatter of the cursors (advanced by one) into token order; cursors that
            // reach the end of the corpus leave the active set
            std::vector<int64_t> pos(hist.begin(), hist.end() - 1);
            std::vector<int32_t> tmp(hi - lo);
            for (int64_t i = lo; i < hi; i++) tmp[pos[corpus[cur[i]]]++] = cur[i];
            for (auto &tn : toks) {
                int64_t a = hist[tn.first], e = hist[tn.first + 1];
                // next-token distribution of this node
                std::vector<int32_t> nt(vocab, 0);
                int64_t before = out;
                for (int64_t i = a; i < e; i++) {
                    int32_t np = tmp[i] + 1;
                    if (np < n) { nt[corpus[np]]++; nxt[out++] = np; }
                }
                for (int t = 0; t < vocab; t++)
                    if (nt[t]) { L.cnt_tok.push_back(t); L.cnt_val.push_back(nt[t]); }
                L.cnt_off.push_back((int64_t)L.cnt_tok.size());
                if (out > before) { nb_node.push_back(tn.second); nb_off.push_back(out); }
            }
        }
        L.n_levels = d + 1;
        cur.swap(nxt);
        n_act = out;
        bnode.swap(nb_node);
        boff.swap(nb_off);
    }
}
}  // namespace

extern "C" int agpt_b200_trie_build(const int32_t *corpus, int64_t n, int max_depth, int subtree_level,
                                    int prune_min_mass, int prune_min_depth, agpt_trie **out) {
    if (!corpus || !out || n < 2 || max_depth < 1) return agpt_set_error(AGPT_E_ARG, "trie_build: bad argument");
    if (n >= (1LL << 31)) return agpt_set_error(AGPT_E_LIMIT, "trie_build: corpus beyond 2^31 tokens");
    int vocab = 0;
    for (int64_t i = 0; i < n; i++) {
        if (corpus[i] < 0) return agpt_set_error(AGPT_E_ARG, "trie_build: negative token");
        vocab = std::max(vocab, corpus[i] + 1);
    }
    Leveled L;
    build_leveled(corpus, n, max_depth, vocab, L);
    if (L.token.size() >= (1ULL << 31)) return agpt_set_error(AGPT_E_LIMIT, "trie_build: more than 2^31 trie nodes");

    agpt_trie *t = new agpt_trie();
    t->leveled_nodes = (int64_t)L.token.size();
    auto push_node = [&](int32_t par, int32_t fcd, int32_t mass, int32_t epd, int32_t key) {
        t->parent.push_back(par); t->first_char_depth.push_back(fcd); t->edge_len.push_back(0);
        t->edge_mass.push_back(mass); t->endpoint_depth.push_back(epd); t->subtree_key.push_back(key);
    };
    push_node(-1, 0, 0, 0, 0);
    t->edge_off.assign(2, 0);
    t->cnt_off.assign(2, 0);
    struct Front { int32_t rid, orig, depth; };
    std::deque<Front> frontier{{0, 0, 1}};
    int32_t max_ep = 0;
    std::vector<int32_t> edge;
    auto mass_of = [&](int32_t id) { int32_t m = 0; for (int64_t e = L.cnt_off[id]; e < L.cnt_off[id + 1]; e++) m += L.cnt_val[e]; return m; };
    while (!frontier.empty()) {
        Front f = frontier.front();
        frontier.pop_front();
        if (f.depth >= L.n_levels) continue;
        for (int32_t c = 0; c < L.child_count[f.orig]; c++) {
            int32_t cur = L.first_child[f.orig] + c, cd = f.depth;
            edge.assign(1, L.token[cur]);
            int32_t mass = mass_of(cur);
            while (L.cnt_off[cur + 1] - L.cnt_off[cur] == 1 && cd + 1 < L.n_levels && L.child_count[cur] == 1) {
                cur = L.first_child[cur]; cd++;
                edge.push_back(L.token[cur]);
            }
            int64_t ec = L.cnt_off[cur + 1] - L.cnt_off[cur];
            if (ec == 0) continue;
            if (mass < prune_min_mass && f.depth >= prune_min_depth) continue;
            int32_t rid = (int32_t)t->parent.size(), key;
            if (subtree_level == 2) {
                if (f.rid == 0) key = (edge[0] << 8) | (edge.size() >= 2 ? edge[1] : 255);
                else {
                    int32_t pk = t->subtree_key[f.rid];
                    key = ((pk & 0xff) != 255) ? pk : ((((pk >> 8) & 0xff) << 8) | edge[0]);
                }
            } else key = f.rid == 0 ? rid : t->subtree_key[f.rid];
            push_node(f.rid, f.depth, mass, cd, key);
            t->edge_len[rid] = (int32_t)edge.size();
            t->edge_tok.insert(t->edge_tok.end(), edge.begin(), edge.end());
            t->edge_off.push_back((int64_t)t->edge_tok.size());
            for (int64_t e = L.cnt_off[cur]; e < L.cnt_off[cur + 1]; e++) { t->cnt_tok.push_back(L.cnt_tok[e]); t->cnt_val.push_back(L.cnt_val[e]); }
            t->cnt_off.push_back((int64_t)t->cnt_tok.size());
            max_ep = std::max(max_ep, cd);
            if (ec >= 2) frontier.push_back({rid, cur, cd + 1});
        }
    }
    t->radix_count = (int32_t)t->parent.size();
    t->n_depth_files = max_ep + 1;
    t->total_edge_chars = (int64_t)t->edge_tok.size();
    t->finish_char_positions();
    *out = t;
    return AGPT_OK;
}

extern "C" void agpt_b200_trie_free(agpt_trie *t) { delete t; }

extern "C" int agpt_b200_trie_info(const agpt_trie *t, agpt_trie_info *o) {
    if (!t || !o) return agpt_set_error(AGPT_E_ARG, "trie_info: null");
    o->radix_count = t->radix_count; o->n_depth_files = t->n_depth_files;
    o->total_edge_chars = t->total_edge_chars; o->total_counts = (int64_t)t->cnt_tok.size();
    o->leveled_nodes = t->leveled_nodes;
    o->parent = t->parent.data(); o->first_char_depth = t->first_char_depth.data(); o->edge_len = t->edge_len.data();
    o->edge_mass = t->edge_mass.data(); o->endpoint_depth = t->endpoint_depth.data(); o->subtree_key = t->subtree_key.data();
    o->edge_off = t->edge_off.data(); o->edge_tok = t->edge_tok.data();
    o->cnt_off = t->cnt_off.data(); o->cnt_tok = t->cnt_tok.data(); o->cnt_val = t->cnt_val.data();
    o->edge_start = t->edge_start.data();
    return AGPT_OK;
}

extern "C" uint64_t agpt_b200_token_hash(const int32_t *tok, int64_t n) {
    uint64_t h = 1469598103934665603ULL;
    const uint64_t prime = 1099511628211ULL;
    for (int64_t i = 0; i < n; i++) {
        uint32_t v = (uint32_t)tok[i];
        for (int b = 0; b < 32; b += 8) { h ^= (v >> b) & 0xFFu; h *= prime; }
    }
    h ^= (uint64_t)n;
    return h * prime;
}

namespace {
const uint32_t RADIX_MAGIC = 0x52445841u;
struct Writer {
    FILE *f = nullptr;
    explicit Writer(const std::string &p) { f = fopen(p.c_str(), "wb"); }
    ~Writer() { if (f) fclose(f); }
    void i32(int32_t v) { fwrite(&v, 4, 1, f); }
    void u32(uint32_t v) { fwrite(&v, 4, 1, f); }
    void i64(int64_t v) { fwrite(&v, 8, 1, f); }
    void u64(uint64_t v) { fwrite(&v, 8, 1, f); }
};
void write_record(Writer &w, const agpt_trie *t, int32_t r) {
    w.i32(r); w.i32(t->parent[r]); w.i32(t->first_char_depth[r]); w.i32(t->edge_len[r]);
    fwrite(t->edge_tok.data() + t->edge_off[r], 4, (size_t)t->edge_len[r], w.f);
    w.i32(t->edge_mass[r]);
    int32_t ec = (int32_t)(t->cnt_off[r + 1] - t->cnt_off[r]);
    w.i32(ec);
    for (int64_t e = t->cnt_off[r]; e < t->cnt_off[r + 1]; e++) { w.i32(t->cnt_tok[e]); w.i32(t->cnt_val[e]); }
}
}  // namespace

extern "C" int agpt_b200_trie_save_dir(const agpt_trie *t, const char *dir, int per_subtree, int32_t corpus_tokens,
                                       int32_t vocab, uint64_t corpus_hash, const char *tag) {
    if (!t || !dir || !tag) return agpt_set_error(AGPT_E_ARG, "trie_save_dir: null");
    std::string d(dir);
    std::vector<std::vector<int32_t>> by_depth(t->n_depth_files);
    for (int32_t r = 1; r < t->radix_count; r++) by_depth[t->endpoint_depth[r]].push_back(r);
    char name[64];
    for (int dd = 0; dd < t->n_depth_files; dd++) {
        snprintf(name, sizeof(name), "/radix_depth_%03d.bin", dd);
        Writer w(d + name);
        if (!w.f) return agpt_set_error(AGPT_E_IO, "cannot write %s%s", dir, name);
        w.u32(RADIX_MAGIC); w.i32(dd); w.i32((int32_t)by_depth[dd].size());
        for (int32_t r : by_depth[dd]) write_record(w, t, r);
    }
    if (per_subtree) {
        std::map<int32_t, std::vector<int32_t>> groups;   // manifest is sorted by key
        for (int32_t r = 1; r < t->radix_count; r++) groups[t->subtree_key[r]].push_back(r);
        Writer m(d + "/manifest.bin");
        if (!m.f) return agpt_set_error(AGPT_E_IO, "cannot write %s/manifest.bin", dir);
        m.u32(RADIX_MAGIC); m.i32(2); m.i32((int32_t)groups.size());
        for (auto &g : groups) {
            int64_t chars = 0; int32_t mx = 0;
            for (int32_t r : g.second) { chars += t->edge_len[r]; mx = std::max(mx, t->endpoint_depth[r]); }
            snprintf(name, sizeof(name), "/subtrees/radix_subtree_%06d.bin", g.first);
            Writer w(d + name);
            if (!w.f) return agpt_set_error(AGPT_E_IO, "cannot write %s%s (does subtrees/ exist?)", dir, name);
            w.u32(RADIX_MAGIC); w.i32(2); w.i32(g.first); w.i32((int32_t)g.second.size()); w.i64(chars); w.i32(mx);
            for (int32_t r : g.second) write_record(w, t, r);
            m.i32(g.first); m.i32((int32_t)g.second.size()); m.i64(chars); m.i32(mx);
        }
    }
    Writer w(d + "/meta.bin");
    if (!w.f) return agpt_set_error(AGPT_E_IO, "cannot write %s/meta.bin", dir);
    w.u32(RADIX_MAGIC); w.i32(2); w.i32(t->radix_count); w.i32(t->n_depth_files); w.i64(t->total_edge_chars);
    w.i32(corpus_tokens); w.i32(vocab); w.u64(corpus_hash);
    int32_t tl = (int32_t)strlen(tag);
    w.i32(tl); fwrite(tag, 1, (size_t)tl, w.f);
    return AGPT_OK;
}

extern "C" int agpt_b200_trie_load_dir(const char *dir, agpt_trie **out) {
    if (!dir || !out) return agpt_set_error(AGPT_E_ARG, "trie_load_dir: null");
    std::string d(dir);
    FILE *f = fopen((d + "/meta.bin").c_str(), "rb");
    if (!f) return agpt_set_error(AGPT_E_IO, "cannot open %s/meta.bin", dir);
    uint32_t magic = 0; int32_t ver = 0, rc = 0, ndf = 0; int64_t tec = 0;
    bool ok = fread(&magic, 4, 1, f) == 1 && fread(&ver, 4, 1, f) == 1 && fread(&rc, 4, 1, f) == 1 &&
              fread(&ndf, 4, 1, f) == 1 && fread(&tec, 8, 1, f) == 1;
    fclose(f);
    if (!ok || magic != RADIX_MAGIC) return agpt_set_error(AGPT_E_IO, "%s/meta.bin: bad radix magic", dir);
    if (ver != 2) return agpt_set_error(AGPT_E_IO, "%s/meta.bin: radix format version %d unsupported (need 2)", dir, ver);
    if (rc < 1 || ndf < 0 || tec < 0) return agpt_set_error(AGPT_E_IO, "%s/meta.bin: bad counts", dir);
    agpt_trie *t = new agpt_trie();
    t->radix_count = rc; t->n_depth_files = ndf; t->total_edge_chars = tec;
    t->parent.assign(rc, -1); t->first_char_depth.assign(rc, 0); t->edge_len.assign(rc, 0); t->edge_mass.assign(rc, 0);
    t->endpoint_depth.assign(rc, 0); t->subtree_key.assign(rc, 0);
    // records arrive in file order; edges and counts are re-laid out by radix id
    std::vector<std::vector<int32_t>> edges(rc), ctok(rc), cval(rc);
    char name[64];
    for (int dd = 0; dd < ndf; dd++) {
        snprintf(name, sizeof(name), "/radix_depth_%03d.bin", dd);
        f = fopen((d + name).c_str(), "rb");
        if (!f) continue;   // an absent depth file is an empty one (src/cuda/agpt_train.cu:816)
        int32_t hd[3];
        if (fread(hd, 4, 3, f) != 3 || (uint32_t)hd[0] != RADIX_MAGIC || hd[1] != dd) { fclose(f); delete t; return agpt_set_error(AGPT_E_IO, "%s%s: bad header", dir, name); }
        for (int32_t i = 0; i < hd[2]; i++) {
            int32_t r4[4];
            if (fread(r4, 4, 4, f) != 4 || r4[0] <= 0 || r4[0] >= rc || r4[3] < 0) { fclose(f); delete t; return agpt_set_error(AGPT_E_IO, "%s%s: bad record", dir, name); }
            int32_t r = r4[0];
            t->parent[r] = r4[1]; t->first_char_depth[r] = r4[2]; t->edge_len[r] = r4[3]; t->endpoint_depth[r] = dd;
            edges[r].resize(r4[3]);
            int32_t me[2];
            if (fread(edges[r].data(), 4, (size_t)r4[3], f) != (size_t)r4[3] || fread(me, 4, 2, f) != 2 || me[1] < 0) { fclose(f); delete t; return agpt_set_error(AGPT_E_IO, "%s%s: truncated record", dir, name); }
            t->edge_mass[r] = me[0];
            ctok[r].resize(me[1]); cval[r].resize(me[1]);
            for (int32_t e = 0; e < me[1]; e++) {
                int32_t tv[2];
                if (fread(tv, 4, 2, f) != 2) { fclose(f); delete t; return agpt_set_error(AGPT_E_IO, "%s%s: truncated counts", dir, name); }
                ctok[r][e] = tv[0]; cval[r][e] = tv[1];
            }
        }
        fclose(f);
    }
    t->edge_off.assign(rc + 1, 0); t->cnt_off.assign(rc + 1, 0);
    for (int32_t r = 0; r < rc; r++) {
        t->edge_off[r + 1] = t->edge_off[r] + (int64_t)edges[r].size();
        t->cnt_off[r + 1] = t->cnt_off[r] + (int64_t)ctok[r].size();
        t->edge_tok.insert(t->edge_tok.end(), edges[r].begin(), edges[r].end());
        t->cnt_tok.insert(t->cnt_tok.end(), ctok[r].begin(), ctok[r].end());
        t->cnt_val.insert(t->cnt_val.end(), cval[r].begin(), cval[r].end());
        // unigram subtree key = depth-1 radix ancestor (parents precede children in id order)
        if (r > 0) t->subtree_key[r] = t->parent[r] == 0 ? r : t->subtree_key[t->parent[r]];
    }
    if ((int64_t)t->edge_tok.size() != tec) { delete t; return agpt_set_error(AGPT_E_IO, "%s: edge chars %lld != meta %lld", dir, (long long)t->edge_tok.size(), (long long)tec); }
    t->finish_char_positions();
    *out = t;
    return AGPT_OK;
}

// Per-subtree files (src/cuda/agpt_train.cu:431-493 manifest, :495-669 load_subtree).
extern "C" int64_t agpt_b200_trie_manifest(const char *dir, int64_t cap, int32_t *keys, int32_t *n_nodes, int64_t *edge_chars,
                                           int32_t *max_endpoint_depth) {
    if (!dir) return agpt_set_error(AGPT_E_ARG, "trie_manifest: null");
    std::string d(dir);
    FILE *f = fopen((d + "/manifest.bin").c_str(), "rb");
    if (!f) return agpt_set_error(AGPT_E_IO, "cannot open %s/manifest.bin", dir);
    int32_t hd[3];
    if (fread(hd, 4, 3, f) != 3 || (uint32_t)hd[0] != RADIX_MAGIC || hd[1] != 2 || hd[2] < 0) { fclose(f); return agpt_set_error(AGPT_E_IO, "%s/manifest.bin: bad header", dir); }
    for (int32_t i = 0; i < hd[2]; i++) {
        int32_t kn[2], me; int64_t ch;
        if (fread(kn, 4, 2, f) != 2 || fread(&ch, 8, 1, f) != 1 || fread(&me, 4, 1, f) != 1) { fclose(f); return agpt_set_error(AGPT_E_IO, "%s/manifest.bin: truncated", dir); }
        if (i < cap) {
            if (keys) keys[i] = kn[0];
            if (n_nodes) n_nodes[i] = kn[1];
            if (edge_chars) edge_chars[i] = ch;
            if (max_endpoint_depth) max_endpoint_depth[i] = me;
        }
    }
    fclose(f);
    return hd[2];
}

extern "C" int agpt_b200_trie_load_subtree(const char *dir, int32_t subtree_key, agpt_trie **out) {
    if (!dir || !out) return agpt_set_error(AGPT_E_ARG, "trie_load_subtree: null");
    char name[96];
    snprintf(name, sizeof(name), "/subtrees/radix_subtree_%06d.bin", subtree_key);
    std::string path = std::string(dir) + name;
    FILE *f = fopen(path.c_str(), "rb");
    if (!f) return agpt_set_error(AGPT_E_IO, "cannot open %s", path.c_str());
    int32_t hd[4]; int64_t tec = 0; int32_t max_ep = 0;
    if (fread(hd, 4, 4, f) != 4 || fread(&tec, 8, 1, f) != 1 || fread(&max_ep, 4, 1, f) != 1 || (uint32_t)hd[0] != RADIX_MAGIC || hd[1] != 2 ||
        hd[2] != subtree_key || hd[3] < 0 || tec < 0) { fclose(f); return agpt_set_error(AGPT_E_IO, "%s: bad header", path.c_str()); }
    const int32_t n = hd[3], rc = n + 1;                  // local id 0 = the (virtual) root, records 1..n in file order
    agpt_trie *t = new agpt_trie();
    t->radix_count = rc; t->n_depth_files = max_ep + 1; t->total_edge_chars = tec;
    t->parent.assign(rc, -1); t->first_char_depth.assign(rc, 0); t->edge_len.assign(rc, 0); t->edge_mass.assign(rc, 0);
    t->endpoint_depth.assign(rc, 0); t->subtree_key.assign(rc, subtree_key); t->edge_start.assign(rc, 0);
    t->edge_off.assign(rc + 1, 0); t->cnt_off.assign(rc + 1, 0);
    std::vector<int32_t> global_id(rc, 0), global_parent(rc, 0);
    for (int32_t i = 1; i <= n; i++) {
        int32_t r4[4], me[2];
        if (fread(r4, 4, 4, f) != 4 || r4[3] < 0) { fclose(f); delete t; return agpt_set_error(AGPT_E_IO, "%s: bad record %d", path.c_str(), i); }
        global_id[i] = r4[0]; global_parent[i] = r4[1];
        t->first_char_depth[i] = r4[2]; t->edge_len[i] = r4[3]; t->endpoint_depth[i] = r4[2] + r4[3] - 1;
        t->edge_start[i] = (int32_t)t->edge_tok.size();     // char positions in file order, as the reference numbers them
        const size_t at = t->edge_tok.size();
        t->edge_tok.resize(at + (size_t)r4[3]);
        if (fread(t->edge_tok.data() + at, 4, (size_t)r4[3], f) != (size_t)r4[3] || fread(me, 4, 2, f) != 2 || me[1] < 0) { fclose(f); delete t; return agpt_set_error(AGPT_E_IO, "%s: truncated record %d", path.c_str(), i); }
        t->edge_mass[i] = me[0];
        for (int32_t e = 0; e < me[1]; e++) {
            int32_t tv[2];
            if (fread(tv, 4, 2, f) != 2) { fclose(f); delete t; return agpt_set_error(AGPT_E_IO, "%s: truncated counts", path.c_str()); }
            t->cnt_tok.push_back(tv[0]); t->cnt_val.push_back(tv[1]);
        }
        t->edge_off[i + 1] = (int64_t)t->edge_tok.size();
        t->cnt_off[i + 1] = (int64_t)t->cnt_tok.size();
    }
    fclose(f);
    t->edge_off[1] = 0; t->cnt_off[1] = 0;
    if ((int64_t)t->edge_tok.size() != tec) { delete t; return agpt_set_error(AGPT_E_IO, "%s: edge chars %lld != header %lld", path.c_str(), (long long)t->edge_tok.size(), (long long)tec); }
    // global -> local ids; a parent that is the virtual root or lies outside the file (the depth-1 node of a bigram
    // subtree) becomes the local root
    std::vector<int32_t> order(n);
    std::iota(order.begin(), order.end(), 1);
    std::sort(order.begin(), order.end(), [&](int32_t a, int32_t b) { return global_id[a] < global_id[b]; });
    for (int32_t i = 1; i <= n; i++) {
        const int32_t gp = global_parent[i];
        int32_t lp = 0;
        if (gp != 0) {
            auto it = std::lower_bound(order.begin(), order.end(), gp, [&](int32_t a, int32_t g) { return global_id[a] < g; });
            if (it != order.end() && global_id[*it] == gp) lp = *it;
        }
        t->parent[i] = lp;
    }
    *out = t;
    return AGPT_OK;
}

extern "C" int agpt_b200_trie_char_tree(const agpt_trie *t, int32_t *parent, int32_t *token, int32_t *depth, int32_t *radix_of_char) {
    if (!t) return agpt_set_error(AGPT_E_ARG, "trie_char_tree: null");
    for (int32_t r = 1; r < t->radix_count; r++) {
        int64_t s = t->edge_start[r];
        int32_t L = t->edge_len[r], p = t->parent[r];
        for (int32_t j = 0; j < L; j++) {
            if (parent) parent[s + j] = j > 0 ? (int32_t)(s + j - 1) : (p == 0 ? -1 : t->edge_start[p] + t->edge_len[p] - 1);
            if (token) token[s + j] = t->edge_tok[t->edge_off[r] + j];
            if (depth) depth[s + j] = t->first_char_depth[r] + j;
            if (radix_of_char) radix_of_char[s + j] = r;
        }
    }
    return AGPT_OK;
}

// --------------------------------------------------------------------------------------
// stochastic subtree sampling ("lightning" training units, src/cuda/agpt_train.cu:152-200, :3928-3943, :4060-4241)
// --------------------------------------------------------------------------------------
static inline uint32_t xorshift32(uint32_t *st) {
    uint32_t x = *st;
    x ^= x << 13; x ^= x >> 17; x ^= x << 5;
    *st = x ? x : 1u;
    return *st;
}
static inline float xorshift_unit(uint32_t *st) { return (float)xorshift32(st) / 4294967296.0f; }

// One super-epoch of `steps` samples.  sampler: 1 uniform over radix nodes, 2 uniform over root children, 3 mass-weighted
// walk from the root that stops with probability p_stop per level (never above max_mass when that is > 0), 4 the same
// walk to a leaf.  A sample's training set is its ancestors, then the sampled node and its descendants breadth
// first (sampler 4: the root-to-node path), stably ordered by endpoint depth.  Call with nodes_out == NULL to learn
// the total number of node ids (the generator state is then left untouched), then again to fill.
extern "C" int64_t agpt_b200_lightning_sample(const agpt_trie *t, int sampler, int steps, float p_stop, int64_t max_mass,
                                              uint32_t *rng_state, int32_t *sample_out, int32_t *n_anc_out, int64_t *node_off_out,
                                              double *mass_out, int32_t *nodes_out, int64_t nodes_cap) {
    if (!t || !rng_state || steps < 0 || sampler < 1 || sampler > 4) return agpt_set_error(AGPT_E_ARG, "lightning_sample: bad argument");
    const int32_t R = t->radix_count;
    std::vector<int64_t> coff(R + 1, 0);
    for (int32_t r = 1; r < R; r++) coff[t->parent[r] + 1]++;
    for (int32_t r = 0; r < R; r++) coff[r + 1] += coff[r];
    std::vector<int32_t> child((size_t)std::max<int64_t>(coff[R], 1));
    {
        std::vector<int64_t> pos(coff.begin(), coff.end() - 1);
        for (int32_t r = 1; r < R; r++) child[pos[t->parent[r]]++] = r;
    }
    uint32_t rng = *rng_state;
    auto root_child = [&]() -> int32_t {
        int64_t nc = coff[1] - coff[0];
        return nc > 0 ? child[coff[0] + (int64_t)(xorshift32(&rng) % (uint32_t)nc)] : 0;
    };
    std::vector<int32_t> buf, sorted;
    int64_t total = 0;
    for (int s = 0; s < steps; s++) {
        int32_t pick_r = 0;
        if (sampler == 3 || sampler == 4) {
            const float stop = sampler == 4 ? 0.0f : p_stop;
            int32_t cur = 0;
            for (;;) {
                const bool forced = max_mass > 0 && cur != 0 && (int64_t)t->edge_mass[cur] > max_mass;
                if (cur != 0 && stop > 0.0f && !forced && xorshift_unit(&rng) < stop) break;
                const int64_t cs = coff[cur], ce = coff[cur + 1];
                if (ce == cs) break;
                double tot = 0.0;
                for (int64_t j = cs; j < ce; j++) tot += (double)t->edge_mass[child[j]];
                int64_t pick;
                if (tot <= 0.0) pick = cs + (int64_t)(xorshift32(&rng) % (uint32_t)(ce - cs));
                else {
                    const double u = (double)xorshift_unit(&rng) * tot;
                    double acc = 0.0;
                    pick = ce - 1;
                    for (int64_t j = cs; j < ce; j++) {
                        acc += (double)t->edge_mass[child[j]];
                        if (u <= acc) { pick = j; break; }
                    }
                }
                cur = child[pick];
            }
            pick_r = cur;
        } else if (sampler == 1) {
            if (R > 1) pick_r = 1 + (int32_t)(xorshift32(&rng) % (uint32_t)(R - 1));
        } else pick_r = root_child();
        if (pick_r == 0) pick_r = root_child();
        buf.clear();
        double mass = 0.0;
        int32_t n_anc = 0;
        if (sampler == 4) {
            for (int32_t c = pick_r; c > 0; c = t->parent[c]) { buf.push_back(c); mass += (double)t->edge_mass[c]; }
            std::reverse(buf.begin(), buf.end());
        } else {
            for (int32_t c = t->parent[pick_r]; c > 0; c = t->parent[c]) { buf.push_back(c); mass += (double)t->edge_mass[c]; }
            std::reverse(buf.begin(), buf.end());
            n_anc = (int32_t)buf.size();
            size_t head = buf.size();
            buf.push_back(pick_r);
            mass += (double)t->edge_mass[pick_r];
            while (head < buf.size()) {
                const int32_t c = buf[head++];
                for (int64_t j = coff[c]; j < coff[c + 1]; j++) { buf.push_back(child[j]); mass += (double)t->edge_mass[child[j]]; }
            }
        }
        if (nodes_out) {
            if (total + (int64_t)buf.size() > nodes_cap) return agpt_set_error(AGPT_E_ARG, "lightning_sample: node buffer too small");
            // stable order by endpoint depth
            sorted.assign(buf.begin(), buf.end());
            std::stable_sort(sorted.begin(), sorted.end(), [&](int32_t a, int32_t b) { return t->endpoint_depth[a] < t->endpoint_depth[b]; });
            std::copy(sorted.begin(), sorted.end(), nodes_out + total);
            if (sample_out) sample_out[s] = pick_r;
            if (n_anc_out) n_anc_out[s] = n_anc;
            if (mass_out) mass_out[s] = mass;
            if (node_off_out) { node_off_out[s] = total; node_off_out[s + 1] = total + (int64_t)buf.size(); }
        }
        total += (int64_t)buf.size();
    }
    if (nodes_out) *rng_state = rng;
    return total;
}

// learning-rate schedule of the trainer (src/cuda/agpt_train.cu:146-216): schedule 0 constant, 1 cosine, 2 linear
// warm-up over warmup_steps then cosine; `step` counts the optimizer steps already taken
extern "C" float agpt_b200_compute_lr(float base_lr, int step, int total_steps, int warmup_steps, int schedule) {
    if (total_steps <= 1 || schedule == 0) return base_lr;
    if (schedule == 2 && step < warmup_steps) return base_lr * ((float)(step + 1) / (float)warmup_steps);
    const int cos_start = schedule == 2 ? warmup_steps : 0;
    if (total_steps <= cos_start) return base_lr;
    float progress = (float)(step - cos_start) / (float)(total_steps - cos_start);
    if (progress > 1.0f) progress = 1.0f;
    return 0.5f * base_lr * (1.0f + cosf(3.14159265358979323846f * progress));
}

// --------------------------------------------------------------------------------------
// per-query mass weights of a launch (host loop of src/cuda/agpt_train.cu:4608-4637, with the mean taken per unit)
// --------------------------------------------------------------------------------------
extern "C" int agpt_b200_mass_weights(const int32_t *edge_mass, const int32_t *edge_len, const int32_t *unit_of_node,
                                      const uint8_t *counted, int64_t n_nodes, int64_t n_units, int mode, float *out_per_query) {
    if (!edge_mass || !edge_len || !out_per_query || n_nodes < 0 || n_units < 1 || mode < 0 || mode > 3)
        return agpt_set_error(AGPT_E_ARG, "mass_weights: bad argument");
    std::vector<float> w((size_t)n_nodes);
    std::vector<double> tot((size_t)n_units, 0.0), tq((size_t)n_units, 0.0);
    for (int64_t i = 0; i < n_nodes; i++) {
        const float c = (float)edge_mass[i];
        w[i] = mode == 1 ? logf(1.0f + c) : mode == 2 ? sqrtf(c) : mode == 3 ? c : 1.0f;
        const int64_t u = unit_of_node ? unit_of_node[i] : 0;
        if (u < 0 || u >= n_units) return agpt_set_error(AGPT_E_ARG, "mass_weights: unit %lld of node %lld out of range", (long long)u, (long long)i);
        if (edge_len[i] < 0) return agpt_set_error(AGPT_E_ARG, "mass_weights: negative edge length");
        if (!counted || counted[i]) { tot[u] += (double)w[i] * edge_len[i]; tq[u] += (double)edge_len[i]; }
    }
    int64_t q = 0;
    for (int64_t i = 0; i < n_nodes; i++) {
        const int64_t u = unit_of_node ? unit_of_node[i] : 0;
        float mean = tq[u] > 0 ? (float)(tot[u] / tq[u]) : 1.0f;
        if (mean <= 0.0f) mean = 1.0f;
        const float v = w[i] / mean;
        for (int32_t j = 0; j < edge_len[i]; j++) out_per_query[q++] = v;
    }
    return AGPT_OK;
}

// --------------------------------------------------------------------------------------
// walker plan
// --------------------------------------------------------------------------------------
extern "C" int agpt_b200_plan_create(const int32_t *parent, int64_t n, int tile_m, int device, agpt_plan **out) {
    if (!parent || !out || n <= 0) return agpt_set_error(AGPT_E_ARG, "plan_create: bad argument");
    if (n >= (1LL << 31) - 256) return agpt_set_error(AGPT_E_LIMIT, "plan_create: more than 2^31 nodes in one plan");
    if (tile_m != 32 && tile_m != 64 && tile_m != 128) return agpt_set_error(AGPT_E_ARG, "plan_create: tile_m must be 32, 64 or 128");
    bool monotone = true;                       // every parent precedes its children (level-order and trie numberings)
    for (int64_t i = 0; i < n; i++) {
        int32_t p = parent[i];
        if (p < -1 || p >= n || p == i) return agpt_set_error(AGPT_E_ARG, "plan_create: parent[%lld]=%d out of range", (long long)i, p);
        if (p >= i) monotone = false;
    }
    agpt_plan *P = new agpt_plan();
    P->n = n; P->tile_m = tile_m;
    P->dfs_to_node.resize(n); P->node_to_dfs.assign(n, -1); P->parent_dfs.resize(n); P->depth.resize(n); P->sub_end.resize(n);
    P->n_groups = 0; P->sum_group_prefix = 0;
    if (monotone) {
        // No stack walk: subtree sizes by one sweep from the last node to the first, then pre-order positions by one
        // sweep forward -- a node's position is its parent's next free slot, siblings arriving in increasing id order.
        std::vector<int32_t> size(n, 1), next_free(n);
        for (int64_t i = n - 1; i >= 0; i--)
            if (parent[i] >= 0) size[parent[i]] += size[i];
        int64_t root_cursor = 0;
        bool any_root = false;
        for (int64_t i = 0; i < n; i++) {
            const int32_t p = parent[i];
            int32_t at;
            if (p < 0) { at = (int32_t)root_cursor; root_cursor += size[i]; any_root = true; }
            else { at = next_free[p]; next_free[p] += size[i]; }
            next_free[i] = at + 1;
            P->node_to_dfs[i] = at;
            P->dfs_to_node[at] = (int32_t)i;
            P->parent_dfs[at] = p < 0 ? -1 : P->node_to_dfs[p];
            P->depth[at] = p < 0 ? 1 : P->depth[P->node_to_dfs[p]] + 1;
            P->sub_end[at] = at + size[i];
        }
        P->n_groups = any_root ? 1 : 0;
        for (int64_t i = 0; i < n; i++)
            if (size[i] > 1) { P->n_groups++; P->sum_group_prefix += P->depth[P->node_to_dfs[i]]; }
    } else {
        // children lists (increasing id order) by counting sort on the parent
        std::vector<int64_t> coff(n + 2, 0);
        for (int64_t i = 0; i < n; i++) coff[parent[i] + 2]++;
        for (int64_t i = 0; i <= n; i++) coff[i + 1] += coff[i];
        std::vector<int32_t> child(n);
        {
            std::vector<int64_t> pos(coff.begin(), coff.end() - 1);
            for (int64_t i = 0; i < n; i++) child[pos[parent[i] + 1]++] = (int32_t)i;
        }
        // iterative pre-order walk; slot -1 (index 0 of coff) is the key-less root
        std::vector<std::pair<int32_t, int64_t>> stack;   // (node, next child cursor)
        stack.reserve(256);
        int64_t pos = 0;
        for (int64_t rc = coff[0]; rc < coff[1]; rc++) {
            stack.clear();
            int32_t root = child[rc];
            auto visit = [&](int32_t v, int32_t par_pos, int32_t dep) {
                P->dfs_to_node[pos] = v; P->node_to_dfs[v] = (int32_t)pos; P->parent_dfs[pos] = par_pos; P->depth[pos] = dep;
                pos++;
                stack.emplace_back(v, coff[v + 1]);
            };
            visit(root, -1, 1);
            while (!stack.empty()) {
                auto &top = stack.back();
                int32_t v = top.first;
                if (top.second < coff[v + 2]) {
                    int32_t c = child[top.second++];
                    int32_t vp = P->node_to_dfs[v];
                    visit(c, vp, P->depth[vp] + 1);
                } else {
                    P->sub_end[P->node_to_dfs[v]] = (int32_t)pos;
                    stack.pop_back();
                }
            }
        }
        if (pos != n) { delete P; return agpt_set_error(AGPT_E_ARG, "plan_create: parent array has a cycle or unreachable nodes (%lld of %lld reached)", (long long)pos, (long long)n); }
        // sibling groups (for the bytes model): one per node with children, plus the root's
        P->n_groups = coff[1] > coff[0] ? 1 : 0;
        for (int64_t v = 0; v < n; v++)
            if (coff[v + 2] > coff[v + 1]) { P->n_groups++; P->sum_group_prefix += P->depth[P->node_to_dfs[v]]; }
    }
    P->max_depth = 0; P->sum_depth = 0;
    for (int64_t i = 0; i < n; i++) { P->max_depth = std::max(P->max_depth, P->depth[i]); P->sum_depth += P->depth[i]; }
    // tiles: chain of the first query of each tile, root side first
    P->n_tiles = (n + tile_m - 1) / tile_m;
    P->chain_off.assign(P->n_tiles + 1, 0);
    for (int64_t t = 0; t < P->n_tiles; t++) P->chain_off[t + 1] = P->chain_off[t] + (P->depth[t * tile_m] - 1);
    P->chain_ids.resize(P->chain_off[P->n_tiles]);
    for (int64_t t = 0; t < P->n_tiles; t++) {
        int32_t a = P->parent_dfs[t * tile_m];
        for (int64_t j = P->chain_off[t + 1] - 1; j >= P->chain_off[t]; j--) { P->chain_ids[j] = a; a = P->parent_dfs[a]; }
    }
    P->chain_end.resize(P->chain_ids.size());
    for (size_t j = 0; j < P->chain_ids.size(); j++) P->chain_end[j] = P->sub_end[P->chain_ids[j]];
    // reduction work list: node a receives one partial row from every tile that starts strictly inside
    // its subtree, i.e. tiles (a / M, (sub_end[a] - 1) / M]; long ranges are cut into segments
    const int64_t SEG = AGPT_REDUCE_SEG;
    for (int64_t a = 0; a < n; a++) {
        int64_t t0 = a / tile_m + 1, t1 = (P->sub_end[a] - 1) / tile_m;   // inclusive range [t0, t1]
        if (t1 < t0) continue;
        int64_t nseg = (t1 - t0 + 1 + SEG - 1) / SEG;
        if (nseg > 1) { P->multi_node.push_back((int32_t)a); P->multi_first.push_back((int64_t)P->n_multi_items); P->multi_count.push_back((int32_t)nseg); }
        for (int64_t s = 0; s < nseg; s++) {
            P->item_node.push_back((int32_t)a);
            P->item_t0.push_back((int32_t)(t0 + s * SEG));
            P->item_t1.push_back((int32_t)std::min(t1, t0 + (s + 1) * SEG - 1));
            P->item_slot.push_back(nseg > 1 ? (int32_t)(P->n_multi_items++) : -1);
        }
        P->n_reduce_nodes++;
    }
    {   // items ordered by their last tile (stable: a counting sort over the tiles), so that "every item whose tiles
        // are all done" is a prefix of the list
        const size_t ni = P->item_node.size();
        std::vector<int64_t> start(P->n_tiles + 1, 0);
        for (size_t i = 0; i < ni; i++) start[P->item_t1[i] + 1]++;
        for (int64_t t = 0; t < P->n_tiles; t++) start[t + 1] += start[t];
        std::vector<int64_t> ord(ni);
        for (size_t i = 0; i < ni; i++) ord[start[P->item_t1[i]]++] = (int64_t)i;
        auto permute = [&](std::vector<int32_t> &v) { std::vector<int32_t> w(v.size()); for (size_t i = 0; i < ord.size(); i++) w[i] = v[ord[i]]; v.swap(w); };
        permute(P->item_node); permute(P->item_t0); permute(P->item_t1); permute(P->item_slot);
    }
    P->device = -1;
    if (device >= 0) {
        int rc = agpt_plan_upload(P, device);
        if (rc != AGPT_OK) { delete P; return rc; }
    }
    *out = P;
    return AGPT_OK;
}

extern "C" int agpt_b200_plan_info(const agpt_plan *p, agpt_plan_info *o) {
    if (!p || !o) return agpt_set_error(AGPT_E_ARG, "plan_info: null");
    o->n = p->n; o->tile_m = p->tile_m; o->n_tiles = p->n_tiles; o->chain_rows = (int64_t)p->chain_ids.size();
    o->max_depth = p->max_depth; o->sum_depth = p->sum_depth; o->sum_group_prefix = p->sum_group_prefix; o->n_groups = p->n_groups;
    o->n_reduce_items = (int64_t)p->item_node.size(); o->n_reduce_nodes = p->n_reduce_nodes; o->n_reduce_multi = (int64_t)p->multi_node.size();
    o->dfs_to_node = p->dfs_to_node.data(); o->node_to_dfs = p->node_to_dfs.data(); o->parent_dfs = p->parent_dfs.data();
    o->depth = p->depth.data(); o->sub_end = p->sub_end.data(); o->device = p->device;
    return AGPT_OK;
}

// --------------------------------------------------------------------------------------
// launch groups: this rank's units packed, in depth-first order, into forests of at most group_rows rows
// (the chunker of src/cuda/agpt_train.cu:4424-4443, on units instead of radix-node counts)
// --------------------------------------------------------------------------------------
struct agpt_groups {
    struct Group { std::vector<int32_t> parent, unit_of_row; std::vector<int64_t> row; std::vector<uint8_t> trained; int32_t n_units = 0; };
    std::vector<Group> groups;
};

extern "C" int agpt_b200_groups_create(const agpt_plan *p, const int64_t *unit_begin, const int64_t *unit_end, const int32_t *unit_rank,
                                       int64_t n_units, int rank, int64_t group_rows, agpt_groups **out) {
    if (!p || !unit_begin || !unit_end || !out || n_units < 0 || group_rows < 1) return agpt_set_error(AGPT_E_ARG, "groups_create: bad argument");
    agpt_groups *G = new agpt_groups();
    agpt_groups::Group cur;
    auto flush = [&]() {
        if (!cur.row.empty()) { G->groups.push_back(std::move(cur)); cur = agpt_groups::Group(); }
    };
    std::vector<int64_t> chain;
    for (int64_t u = 0; u < n_units; u++) {
        if (unit_rank && unit_rank[u] != rank) continue;
        const int64_t b = unit_begin[u], e = unit_end[u];
        if (b < 0 || e > p->n || b >= e) { delete G; return agpt_set_error(AGPT_E_ARG, "groups_create: unit %lld has a bad range", (long long)u); }
        // a unit that does not start at depth 1 carries its ancestors as context rows (attended, not trained), so every
        // chain is complete and results do not depend on the partition
        chain.clear();
        for (int64_t a = p->parent_dfs[b]; a >= 0; a = p->parent_dfs[a]) chain.push_back(a);
        std::reverse(chain.begin(), chain.end());
        const int64_t k = (int64_t)chain.size(), rows = k + (e - b);
        if (!cur.row.empty() && (int64_t)cur.row.size() + rows > group_rows) flush();
        const int64_t off = (int64_t)cur.row.size();
        if (off + rows >= (1LL << 31) - 256) { delete G; return agpt_set_error(AGPT_E_LIMIT, "groups_create: more than 2^31 rows in one group"); }
        const int32_t unit_local = cur.n_units++;
        for (int64_t j = 0; j < k; j++) {
            cur.parent.push_back((int32_t)(j == 0 ? -1 : off + j - 1));
            cur.row.push_back(chain[j]); cur.trained.push_back(0); cur.unit_of_row.push_back(unit_local);
        }
        for (int64_t i = b; i < e; i++) {
            const int64_t pp = p->parent_dfs[i];
            // the unit's first row hangs under its context chain (a root without one); rows inside keep their parent
            const int64_t lp = i == b ? (k ? off + k - 1 : -1) : (pp < b ? -1 : off + k + (pp - b));
            cur.parent.push_back((int32_t)lp);
            cur.row.push_back(i); cur.trained.push_back(1); cur.unit_of_row.push_back(unit_local);
        }
    }
    flush();
    *out = G;
    return AGPT_OK;
}

extern "C" int64_t agpt_b200_groups_count(const agpt_groups *g) { return g ? (int64_t)g->groups.size() : 0; }

extern "C" int agpt_b200_groups_get(const agpt_groups *g, int64_t i, agpt_group_info *o) {
    if (!g || !o || i < 0 || i >= (int64_t)g->groups.size()) return agpt_set_error(AGPT_E_ARG, "groups_get: bad argument");
    const agpt_groups::Group &x = g->groups[i];
    o->n = (int64_t)x.row.size(); o->n_units = x.n_units;
    o->parent = x.parent.data(); o->row = x.row.data(); o->trained = x.trained.data(); o->unit_of_row = x.unit_of_row.data();
    return AGPT_OK;
}

extern "C" void agpt_b200_groups_free(agpt_groups *g) { delete g; }

extern "C" int64_t agpt_b200_attn_bwd_workspace_bytes(const agpt_plan *p, int d_model) {
    if (!p || d_model <= 0) return agpt_set_error(AGPT_E_ARG, "attn_bwd_workspace_bytes: bad argument");
    // partial dK and dV rows of every tile's chain, then the per-segment sums of long reductions
    int64_t rows = (int64_t)p->chain_ids.size() + p->n_multi_items;
    return std::max<int64_t>(256, rows * 2 * (int64_t)d_model * 4);
}

extern "C" int64_t agpt_b200_plan_units(const agpt_plan *p, int level, int64_t cap, int64_t *ub, int64_t *ue) {
    if (!p || (level != 1 && level != 2)) return agpt_set_error(AGPT_E_ARG, "plan_units: bad argument");
    int64_t cnt = 0;
    auto emit = [&](int64_t b, int64_t e) { if (cnt < cap && ub && ue) { ub[cnt] = b; ue[cnt] = e; } cnt++; };
    for (int64_t a = 0; a < p->n; a = p->sub_end[a]) {       // depth-1 nodes
        // a depth-1 node with a single child stays with that child (its radix edge runs on past depth 1)
        if (level == 1 || (a + 1 < p->sub_end[a] && p->sub_end[a + 1] == p->sub_end[a])) { emit(a, p->sub_end[a]); continue; }
        emit(a, a + 1);
        for (int64_t c = a + 1; c < p->sub_end[a]; c = p->sub_end[c]) emit(c, p->sub_end[c]);
    }
    return cnt;
}

extern "C" int agpt_b200_partition_lpt(const int64_t *w, int64_t n_units, int n_ranks, int32_t *rank_of_unit) {
    if (!w || !rank_of_unit || n_units < 0 || n_ranks < 1) return agpt_set_error(AGPT_E_ARG, "partition_lpt: bad argument");
    std::vector<int64_t> order(n_units), load(n_ranks, 0);
    std::iota(order.begin(), order.end(), 0);
    std::stable_sort(order.begin(), order.end(), [&](int64_t a, int64_t b) { return w[a] > w[b]; });
    for (int64_t u : order) {
        int best = 0;
        for (int r = 1; r < n_ranks; r++) if (load[r] < load[best]) best = r;
        rank_of_unit[u] = best;
        load[best] += w[u];
    }
    return AGPT_OK;
}
