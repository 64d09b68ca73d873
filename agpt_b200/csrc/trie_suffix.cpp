// Radix-trie construction from a suffix order.
//
// The level-by-level builder in host_trie.cpp (the reference's two-stage build, src/agpt/streaming_leveled_builder.cr:31-118
// then src/agpt/streaming_radix_builder.cr:103-343) spends its time refining buckets of suffix start positions, one
// level at a time: O(n * depth) random accesses on one host thread.  That part is a sort.  Here the start positions
// 0..n-2 arrive already ordered by their first max_depth+1 tokens (positions past the end of the corpus order before
// every token), together with the common-prefix length of each neighbouring pair -- produced on the GPU by
// trie_gpu.cu -- and the trie is assembled from that in one linear pass:
//
//   * a prefix is a radix node's endpoint iff it has two or more distinct next tokens, or it has depth max_depth
//     and at least one next token; in the ordered list a prefix is an interval, its next tokens are the runs
//     between the places where the neighbours' common prefix equals its depth (the classic LCP-interval tree);
//   * the reference numbers radix nodes in the order its breadth-first frontier emits them: level by level (level =
//     number of radix ancestors), and inside a level in (parent id, token) order, which is the left-to-right order
//     of the intervals; so ids are a stable counting sort of the emission order by level;
//   * edge mass is the number of suffixes that continue past the first character of the edge; pruning
//     (mass < prune_min_mass at first-character depth >= prune_min_depth) removes a node with its subtree.
//
// The result is identical, array for array, to agpt_b200_trie_build (tests compare them on random corpora,
// including the effects of the corpus end, where a suffix stops before max_depth).
#include <algorithm>
#include <cstdint>
#include <vector>

#include "../../include/agpt_b200.h"
#include "internal.h"

namespace {

struct Endpoint {
    int32_t lb, rb;        // interval of ordered suffixes that share the endpoint's prefix
    int32_t depth;         // endpoint depth
    int32_t last_split;    // last place inside (lb, rb] where the neighbours' common prefix equals depth; -1: one run
    int32_t parent;        // emission index of the enclosing endpoint, -1: the root
};

struct Open {              // an open interval of the LCP-interval tree
    int32_t lcp, lb, last_split, n_splits;
};

}  // namespace

extern "C" int agpt_b200_trie_from_suffix_order(const int32_t *corpus, int64_t n, int max_depth, int subtree_level, int prune_min_mass,
                                                int prune_min_depth, const int32_t *sa, const int32_t *lcp, agpt_trie **out) {
    if (!corpus || !sa || !lcp || !out || max_depth < 1) return agpt_set_error(AGPT_E_ARG, "trie_from_suffix_order: bad argument");
    if (n < (int64_t)max_depth + 2) return agpt_set_error(AGPT_E_ARG, "trie_from_suffix_order: corpus shorter than max_depth + 2 tokens");
    if (n >= (1LL << 31)) return agpt_set_error(AGPT_E_LIMIT, "trie_from_suffix_order: corpus beyond 2^31 tokens");
    const int32_t m = (int32_t)(n - 1);          // suffixes start at 0 .. n-2
    const int D = max_depth, KL = max_depth + 1;   // the order and the common prefixes cover KL tokens
    auto len_of = [&](int32_t i) -> int { int64_t l = n - sa[i]; return l < KL ? (int)l : KL; };
    auto lcp_at = [&](int64_t i) -> int { return (i <= 0 || i >= m) ? 0 : lcp[i]; };

    std::vector<Endpoint> eps;
    std::vector<int32_t> pending;                  // endpoints not yet enclosed by a later (shallower) one
    std::vector<int32_t> prev_split(m, -1);        // chain of split points of one interval, newest first
    auto emit = [&](int32_t lb, int32_t rb, int32_t depth, int32_t last_split) {
        int32_t id = (int32_t)eps.size();
        eps.push_back({lb, rb, depth, last_split, -1});
        while (!pending.empty() && eps[pending.back()].lb >= lb) {
            eps[pending.back()].parent = id;
            pending.pop_back();
        }
        pending.push_back(id);
    };
    std::vector<Open> st;
    st.push_back({0, 0, -1, 0});
    int64_t leveled = 1;
    for (int64_t i = 1; i <= m; i++) {
        const int cur = i < m ? lcp[i] : -1;       // -1 closes everything, the root included
        {
            // the suffix at i-1 alone: a depth-D endpoint with one next token if it is long enough and nothing shares
            // its first D tokens
            const int32_t j = (int32_t)(i - 1);
            const int left = lcp_at(j), right = cur < 0 ? 0 : cur;
            if (len_of(j) >= KL && std::max(left, right) < D) emit(j, j, D, -1);
            leveled += std::min(len_of(j), D) - std::min(left, D);
        }
        int32_t lb = (int32_t)(i - 1);
        while (!st.empty() && st.back().lcp > cur) {
            const Open iv = st.back();
            st.pop_back();
            const int32_t rb = (int32_t)(i - 1);
            lb = iv.lb;
            if (iv.lcp == 0) break;                // the root
            if (iv.lcp >= KL) {
                // every suffix of the interval shares the next token too: the depth-D prefix is an endpoint of its own
                // only if the enclosing interval splits above depth D
                if (std::max(lcp_at(iv.lb), cur < 0 ? 0 : cur) < D) emit(iv.lb, rb, D, -1);
                continue;
            }
            // next tokens = runs between the split points; a suffix that ends exactly here (it orders first) has none
            const int real = 1 + iv.n_splits - (len_of(iv.lb) == iv.lcp ? 1 : 0);
            if (iv.lcp < D ? real >= 2 : real >= 1) emit(iv.lb, rb, iv.lcp, iv.last_split);
        }
        if (cur >= 0) {
            if (!st.empty() && st.back().lcp == cur) {
                prev_split[i] = st.back().last_split;
                st.back().last_split = (int32_t)i;
                st.back().n_splits++;
            } else {
                st.push_back({cur, lb, (int32_t)i, 1});
            }
        }
    }

    const int32_t E = (int32_t)eps.size();
    // parents come after their children in emission order: walk backwards for level, first-character depth, mass, pruning
    std::vector<int32_t> level(E), fcd(E), mass(E);
    std::vector<uint8_t> pruned(E);
    int32_t max_level = 0;
    for (int32_t e = E - 1; e >= 0; e--) {
        const Endpoint &x = eps[e];
        level[e] = x.parent < 0 ? 1 : level[x.parent] + 1;
        fcd[e] = x.parent < 0 ? 1 : eps[x.parent].depth + 1;
        // suffixes sharing the first fcd tokens: the interval, plus suffixes to its left that end inside the edge
        int32_t lbx = x.lb;
        while (lbx > 0 && lcp[lbx] >= fcd[e]) lbx--;
        mass[e] = (x.rb - lbx + 1) - (len_of(lbx) == fcd[e] ? 1 : 0);
        pruned[e] = (x.parent >= 0 && pruned[x.parent]) || (mass[e] < prune_min_mass && fcd[e] >= prune_min_depth);
        if (!pruned[e]) max_level = std::max(max_level, level[e]);
    }
    // breadth-first ids: counting sort of the emission order by level
    std::vector<int32_t> level_off(max_level + 2, 0), id(E, -1);
    for (int32_t e = 0; e < E; e++)
        if (!pruned[e]) level_off[level[e] + 1]++;
    for (int l = 0; l <= max_level; l++) level_off[l + 1] += level_off[l];
    int32_t R = 1;
    for (int32_t e = 0; e < E; e++)
        if (!pruned[e]) { id[e] = 1 + level_off[level[e]]++; R++; }

    agpt_trie *t = new agpt_trie();
    t->radix_count = R;
    t->leveled_nodes = leveled;
    t->parent.assign(R, -1);
    t->first_char_depth.assign(R, 0);
    t->edge_len.assign(R, 0);
    t->edge_mass.assign(R, 0);
    t->endpoint_depth.assign(R, 0);
    t->subtree_key.assign(R, 0);
    t->edge_off.assign(R + 1, 0);
    t->cnt_off.assign(R + 1, 0);
    std::vector<int32_t> ep_of(R, -1);             // endpoint of each radix id
    int32_t max_ep = 0;
    for (int32_t e = 0; e < E; e++) {
        if (pruned[e]) continue;
        const Endpoint &x = eps[e];
        const int32_t r = id[e];
        ep_of[r] = e;
        t->parent[r] = x.parent < 0 ? 0 : id[x.parent];
        t->first_char_depth[r] = fcd[e];
        t->edge_len[r] = x.depth - fcd[e] + 1;
        t->edge_mass[r] = mass[e];
        t->endpoint_depth[r] = x.depth;
        max_ep = std::max(max_ep, x.depth);
        // count entries: one per run of the interval that has a next token
        int32_t entries;
        if (x.last_split < 0) entries = 1;
        else {
            entries = 1;
            for (int32_t s = x.last_split; s >= 0; s = prev_split[s]) entries++;
            if (len_of(x.lb) == x.depth) entries--;
        }
        t->edge_off[r + 1] = t->edge_len[r];
        t->cnt_off[r + 1] = entries;
    }
    for (int32_t r = 0; r < R; r++) { t->edge_off[r + 1] += t->edge_off[r]; t->cnt_off[r + 1] += t->cnt_off[r]; }
    t->edge_tok.resize((size_t)t->edge_off[R]);
    t->cnt_tok.resize((size_t)t->cnt_off[R]);
    t->cnt_val.resize((size_t)t->cnt_off[R]);
    std::vector<int32_t> splits;
    for (int32_t r = 1; r < R; r++) {
        const Endpoint &x = eps[ep_of[r]];
        const int32_t f = t->first_char_depth[r], el = t->edge_len[r];
        const int32_t *src = corpus + sa[x.rb] + f - 1;     // the last suffix of the interval is as long as any
        std::copy(src, src + el, t->edge_tok.begin() + t->edge_off[r]);
        int64_t c = t->cnt_off[r];
        if (x.last_split < 0) {
            t->cnt_tok[c] = corpus[(int64_t)sa[x.rb] + x.depth];
            t->cnt_val[c] = x.rb - x.lb + 1;
        } else {
            splits.clear();
            for (int32_t s = x.last_split; s >= 0; s = prev_split[s]) splits.push_back(s);
            int32_t a = x.lb;
            for (int k = (int)splits.size(); k >= 0; k--) {           // runs in order: [a, next split)
                const int32_t b = k > 0 ? splits[k - 1] : x.rb + 1;
                if (len_of(a) > x.depth) {
                    t->cnt_tok[c] = corpus[(int64_t)sa[a] + x.depth];
                    t->cnt_val[c] = b - a;
                    c++;
                }
                a = b;
            }
        }
        // subtree key (src/agpt/streaming_radix_builder.cr:215-240): the root child, or the first two characters
        const int32_t par = t->parent[r];
        const int32_t e0 = t->edge_tok[t->edge_off[r]];
        int32_t key;
        if (subtree_level == 2) {
            if (par == 0) key = (e0 << 8) | (el >= 2 ? t->edge_tok[t->edge_off[r] + 1] : 255);
            else {
                const int32_t pk = t->subtree_key[par];
                key = ((pk & 0xff) != 255) ? pk : ((((pk >> 8) & 0xff) << 8) | e0);
            }
        } else key = par == 0 ? r : t->subtree_key[par];
        t->subtree_key[r] = key;
    }
    t->n_depth_files = max_ep + 1;
    t->total_edge_chars = (int64_t)t->edge_tok.size();
    t->finish_char_positions();
    *out = t;
    return AGPT_OK;
}
