/*
 * agpt_oracle.c — CPU restatement of the AGPT trie-walk hot path.
 *
 * TEST INFRASTRUCTURE ONLY.  This file is the checker for the CUDA library: the
 * parity tests, the smoke check and the CPU-baseline leg of the benchmark call it;
 * nothing on the product path does.  It is a plain-C restatement, written from
 * scratch, of the algorithms in the reference project (paths are relative to the
 * reference project's root):
 *
 *   leveled trie build        src/agpt/streaming_leveled_builder.cr:31-118
 *   radix trie build          src/agpt/streaming_radix_builder.cr:103-343
 *   radix dir writer          src/agpt/streaming_radix_builder.cr:388-451
 *   char positions/ancestors  src/cuda/agpt_train.cu:772-946
 *   corpus hash               src/agpt/trie_corpus.cr:120-134
 *   RoPE table / apply        src/cuda/agpt_train.cu:2298-2321, :1305-1351;
 *                             src/agpt/batched_depth_forward.cr:1051-1061
 *   per-node attention        src/agpt/batched_depth_forward.cr:973-1023
 *   sibling-grouped attention src/agpt/batched_depth_forward.cr:836-971
 *   attention backward        src/agpt/batched_depth_backward.cr:605-695
 *   matrix-form backward      spec/agpt_backward_attention_spec.cr:185-276
 *   per-query loss            src/cuda/agpt_train.cu:2069-2197
 *   per-node loss (leveled)   src/cuda/agpt_train.cu:1947-2029
 *   per-node loss (Crystal)   src/agpt/trie_walk_trainer.cr:118-158
 *   chunk mass weights        src/cuda/agpt_train.cu:4608-4637
 *   packed-prefix layout      src/agpt/batched_depth_forward.cr:656-801,
 *                             src/cuda/agpt_train.cu:4445-4483
 *
 * Parity status: the attention kernels of the reference's GPU path live in an
 * un-vendored dependency (shard trans/microgpt, 0.2.0+git.commit.bdd8e82e...), so
 * for those symbols parity is pinned only by the reference's own formula-equivalence
 * spec (two formulas agree to 1e-5) and by trie-shape anchors; there are no stored
 * numeric vectors in the reference for logits, loss or gradients.
 *
 * Tree convention used by the attention functions: nodes 0..n-1, parent[i] == -1
 * for a child of the (key-less) root, otherwise parent[i] < i.  Row i of q/k/v is
 * the post-RoPE projection of node i; heads are contiguous slices of the row.
 */
#include <math.h>
#include <stdint.h>
#include <stdio.h>
#include <stdlib.h>
#include <string.h>
#ifdef _OPENMP
#include <omp.h>
#endif

#define ORC_API __attribute__((visibility("default")))

/* ------------------------------------------------------------------------- */
/* corpus hash: FNV-1a over 4 LE bytes per token, then the size              */
/* (src/agpt/trie_corpus.cr:120-134)                                         */
/* ------------------------------------------------------------------------- */
ORC_API uint64_t orc_token_hash(const int32_t *tok, int64_t n) {
    uint64_t h = 1469598103934665603ULL, prime = 1099511628211ULL;
    for (int64_t i = 0; i < n; i++) {
        uint64_t v = (uint32_t)tok[i];
        for (int b = 0; b < 4; b++) { h ^= v & 0xFF; h *= prime; v >>= 8; }
    }
    h ^= (uint64_t)n;
    h *= prime;
    return h;
}

/* ------------------------------------------------------------------------- */
/* Leveled trie (src/agpt/streaming_leveled_builder.cr:31-118)               */
/* ------------------------------------------------------------------------- */
typedef struct {
    int32_t n_nodes;        /* including root (id 0) */
    int32_t n_levels;       /* depth files 0..n_levels-1 */
    int32_t *parent, *token, *depth;
    int32_t *level_start;   /* [n_levels+1] first id of each depth */
    int64_t *cnt_off;       /* [n_nodes+1] */
    int32_t *cnt_tok, *cnt_val;
    int32_t *first_child, *child_count; /* derived: children are id-contiguous */
} orc_leveled;

typedef struct { int32_t parent, tok, cursor; } orc_act;

static int act_cmp(const void *a, const void *b) {
    const orc_act *x = (const orc_act *)a, *y = (const orc_act *)b;
    if (x->parent != y->parent) return x->parent < y->parent ? -1 : 1;
    if (x->tok != y->tok) return x->tok < y->tok ? -1 : 1;
    if (x->cursor != y->cursor) return x->cursor < y->cursor ? -1 : 1;
    return 0;
}
static int int_cmp(const void *a, const void *b) {
    int32_t x = *(const int32_t *)a, y = *(const int32_t *)b;
    return x < y ? -1 : (x > y);
}

#define GROW(ptr, cap, need, type)                                   \
    do {                                                             \
        if ((int64_t)(need) > (int64_t)(cap)) {                      \
            int64_t nc = (cap) ? (cap) * 2 : 1024;                   \
            while (nc < (int64_t)(need)) nc *= 2;                    \
            (ptr) = (type *)realloc((ptr), (size_t)nc * sizeof(type)); \
            (cap) = nc;                                              \
        }                                                            \
    } while (0)

ORC_API orc_leveled *orc_leveled_build(const int32_t *corpus, int32_t n, int32_t max_depth) {
    orc_leveled *t = (orc_leveled *)calloc(1, sizeof(*t));
    int64_t ncap = 0, ccap = 0, lcap = 0, n_cnt = 0;
    int32_t n_nodes = 0;
    GROW(t->parent, ncap, 1, int32_t);
    t->token = (int32_t *)malloc((size_t)ncap * 4);
    t->depth = (int32_t *)malloc((size_t)ncap * 4);
    t->cnt_off = (int64_t *)malloc((size_t)(ncap + 1) * 8);
    GROW(t->level_start, lcap, max_depth + 3, int32_t);
    /* depth 0: root, no counts (the builder writes an empty entry list for it) */
    t->parent[0] = -1; t->token[0] = -1; t->depth[0] = 0; t->cnt_off[0] = 0; t->cnt_off[1] = 0;
    n_nodes = 1;
    t->level_start[0] = 0; t->level_start[1] = 1;
    int32_t n_levels = 1;

    int64_t n_act = n > 0 ? n - 1 : 0;   /* starts 0..n-2 */
    orc_act *act = (orc_act *)malloc((size_t)(n_act ? n_act : 1) * sizeof(orc_act));
    orc_act *nxt = (orc_act *)malloc((size_t)(n_act ? n_act : 1) * sizeof(orc_act));
    for (int64_t i = 0; i < n_act; i++) { act[i].cursor = (int32_t)i; act[i].parent = 0; }
    int32_t *tmp = (int32_t *)malloc((size_t)(n_act ? n_act : 1) * 4);

    for (int32_t d = 1; n_act > 0 && d <= max_depth; d++) {
        for (int64_t i = 0; i < n_act; i++) act[i].tok = corpus[act[i].cursor];
        qsort(act, (size_t)n_act, sizeof(orc_act), act_cmp);   /* keys sorted by (parent, token) */
        int64_t n_next = 0;
        int64_t i = 0;
        while (i < n_act) {
            int64_t j = i;
            while (j < n_act && act[j].parent == act[i].parent && act[j].tok == act[i].tok) j++;
            int32_t nid = n_nodes++;
            if (n_nodes + 1 > ncap) {
                int64_t oc = ncap; (void)oc;
                GROW(t->parent, ncap, n_nodes + 1, int32_t);
                t->token = (int32_t *)realloc(t->token, (size_t)ncap * 4);
                t->depth = (int32_t *)realloc(t->depth, (size_t)ncap * 4);
                t->cnt_off = (int64_t *)realloc(t->cnt_off, (size_t)(ncap + 1) * 8);
            }
            t->parent[nid] = act[i].parent; t->token[nid] = act[i].tok; t->depth[nid] = d;
            /* next-token distribution, sorted by token */
            int64_t m = 0;
            for (int64_t c = i; c < j; c++) {
                int32_t np = act[c].cursor + 1;
                if (np < n) {
                    tmp[m++] = corpus[np];
                    nxt[n_next].cursor = np; nxt[n_next].parent = nid; n_next++;
                }
            }
            qsort(tmp, (size_t)m, 4, int_cmp);
            int64_t a = 0;
            while (a < m) {
                int64_t b = a;
                while (b < m && tmp[b] == tmp[a]) b++;
                if (n_cnt + 1 > ccap) {
                    GROW(t->cnt_tok, ccap, n_cnt + 1, int32_t);
                    t->cnt_val = (int32_t *)realloc(t->cnt_val, (size_t)ccap * 4);
                }
                t->cnt_tok[n_cnt] = tmp[a]; t->cnt_val[n_cnt] = (int32_t)(b - a); n_cnt++;
                a = b;
            }
            t->cnt_off[nid + 1] = n_cnt;
            i = j;
        }
        t->level_start[d + 1] = n_nodes;
        n_levels = d + 1;
        orc_act *sw = act; act = nxt; nxt = sw;
        n_act = n_next;
    }
    free(act); free(nxt); free(tmp);
    t->n_nodes = n_nodes; t->n_levels = n_levels;
    if (!t->cnt_tok) { t->cnt_tok = (int32_t *)malloc(4); t->cnt_val = (int32_t *)malloc(4); }
    t->first_child = (int32_t *)malloc((size_t)n_nodes * 4);
    t->child_count = (int32_t *)calloc((size_t)n_nodes, 4);
    for (int32_t i = 0; i < n_nodes; i++) t->first_child[i] = -1;
    for (int32_t i = 1; i < n_nodes; i++) {
        int32_t p = t->parent[i];
        if (t->first_child[p] < 0) t->first_child[p] = i;
        t->child_count[p]++;
    }
    return t;
}

ORC_API void orc_leveled_free(orc_leveled *t) {
    if (!t) return;
    free(t->parent); free(t->token); free(t->depth); free(t->level_start);
    free(t->cnt_off); free(t->cnt_tok); free(t->cnt_val); free(t->first_child); free(t->child_count);
    free(t);
}

/* ------------------------------------------------------------------------- */
/* Radix trie from leveled (src/agpt/streaming_radix_builder.cr:103-343)     */
/* ------------------------------------------------------------------------- */
typedef struct {
    int32_t radix_count;          /* including virtual root id 0 */
    int32_t n_depth_files;        /* max_endpoint_depth + 1 */
    int64_t total_edge_chars;
    int32_t *parent, *first_char_depth, *edge_len, *edge_mass, *endpoint_depth, *subtree_key;
    int32_t *endpoint_leveled_id;
    int64_t *edge_off;            /* [radix_count+1] into edge_tok, emission order */
    int32_t *edge_tok;
    int64_t *cnt_off;             /* [radix_count+1] */
    int32_t *cnt_tok, *cnt_val;
    /* char-position index as the trainer's loader derives it
       (src/cuda/agpt_train.cu:809-846, :892-939) */
    int32_t *edge_start;          /* char position of the first edge char, file order */
    int64_t *anc_off;             /* [radix_count+1] */
    int32_t *anc_ids;             /* ancestor char positions, root to leaf */
} orc_radix;

ORC_API orc_radix *orc_radix_build(const orc_leveled *lv, int32_t subtree_level,
                                   int32_t prune_min_mass, int32_t prune_min_depth) {
    orc_radix *r = (orc_radix *)calloc(1, sizeof(*r));
    int64_t cap = 1024, ecap = 4096, ccap = 4096;
    r->parent = (int32_t *)malloc(cap * 4); r->first_char_depth = (int32_t *)malloc(cap * 4);
    r->edge_len = (int32_t *)malloc(cap * 4); r->edge_mass = (int32_t *)malloc(cap * 4);
    r->endpoint_depth = (int32_t *)malloc(cap * 4); r->subtree_key = (int32_t *)malloc(cap * 4);
    r->endpoint_leveled_id = (int32_t *)malloc(cap * 4);
    r->edge_off = (int64_t *)malloc((cap + 1) * 8); r->cnt_off = (int64_t *)malloc((cap + 1) * 8);
    r->edge_tok = (int32_t *)malloc(ecap * 4);
    r->cnt_tok = (int32_t *)malloc(ccap * 4); r->cnt_val = (int32_t *)malloc(ccap * 4);
    /* id 0: virtual root */
    r->parent[0] = -1; r->first_char_depth[0] = 0; r->edge_len[0] = 0; r->edge_mass[0] = 0;
    r->endpoint_depth[0] = 0; r->subtree_key[0] = 0; r->endpoint_leveled_id[0] = 0;
    r->edge_off[0] = 0; r->edge_off[1] = 0; r->cnt_off[0] = 0; r->cnt_off[1] = 0;
    int32_t next_id = 1; int64_t n_edge = 0, n_cnt = 0; int32_t max_ep = 0;

    /* frontier deque of (parent_radix_id, start_original_id, start_char_depth) */
    int64_t fcap = 1024, fhead = 0, ftail = 0;
    int32_t *fr = (int32_t *)malloc(fcap * 3 * 4);
    fr[0] = 0; fr[1] = 0; fr[2] = 1; ftail = 1;
    int32_t *edge = (int32_t *)malloc((size_t)(lv->n_levels + 2) * 4);

    while (fhead < ftail) {
        int32_t parent_rid = fr[fhead * 3], start_orig = fr[fhead * 3 + 1], start_depth = fr[fhead * 3 + 2];
        fhead++;
        if (start_depth >= lv->n_levels) continue;
        int32_t nc = lv->child_count[start_orig];
        if (nc == 0) continue;
        int32_t fc = lv->first_child[start_orig];
        for (int32_t ci = 0; ci < nc; ci++) {
            int32_t cur = fc + ci, cur_depth = start_depth, elen = 0;
            edge[elen++] = lv->token[cur];
            int32_t mass = 0;
            for (int64_t e = lv->cnt_off[cur]; e < lv->cnt_off[cur + 1]; e++) mass += lv->cnt_val[e];
            for (;;) {
                int64_t nce = lv->cnt_off[cur + 1] - lv->cnt_off[cur];
                if (nce == 1 && cur_depth + 1 < lv->n_levels) {
                    if (lv->child_count[cur] != 1) break;
                    cur = lv->first_child[cur]; cur_depth++;
                    edge[elen++] = lv->token[cur];
                } else break;
            }
            int64_t ec = lv->cnt_off[cur + 1] - lv->cnt_off[cur];
            if (ec == 0) continue;                                      /* end-of-corpus leaf */
            if (mass < prune_min_mass && start_depth >= prune_min_depth) continue;
            int32_t rid = next_id++;
            if (next_id + 1 > cap) {
                cap *= 2;
                r->parent = (int32_t *)realloc(r->parent, cap * 4);
                r->first_char_depth = (int32_t *)realloc(r->first_char_depth, cap * 4);
                r->edge_len = (int32_t *)realloc(r->edge_len, cap * 4);
                r->edge_mass = (int32_t *)realloc(r->edge_mass, cap * 4);
                r->endpoint_depth = (int32_t *)realloc(r->endpoint_depth, cap * 4);
                r->subtree_key = (int32_t *)realloc(r->subtree_key, cap * 4);
                r->endpoint_leveled_id = (int32_t *)realloc(r->endpoint_leveled_id, cap * 4);
                r->edge_off = (int64_t *)realloc(r->edge_off, (cap + 1) * 8);
                r->cnt_off = (int64_t *)realloc(r->cnt_off, (cap + 1) * 8);
            }
            while (n_edge + elen > ecap) { ecap *= 2; r->edge_tok = (int32_t *)realloc(r->edge_tok, ecap * 4); }
            while (n_cnt + ec > ccap) {
                ccap *= 2;
                r->cnt_tok = (int32_t *)realloc(r->cnt_tok, ccap * 4);
                r->cnt_val = (int32_t *)realloc(r->cnt_val, ccap * 4);
            }
            r->parent[rid] = parent_rid; r->first_char_depth[rid] = start_depth;
            r->edge_len[rid] = elen; r->edge_mass[rid] = mass; r->endpoint_depth[rid] = cur_depth;
            r->endpoint_leveled_id[rid] = cur;
            memcpy(r->edge_tok + n_edge, edge, (size_t)elen * 4); n_edge += elen;
            r->edge_off[rid + 1] = n_edge;
            for (int64_t e = 0; e < ec; e++) {
                r->cnt_tok[n_cnt + e] = lv->cnt_tok[lv->cnt_off[cur] + e];
                r->cnt_val[n_cnt + e] = lv->cnt_val[lv->cnt_off[cur] + e];
            }
            n_cnt += ec; r->cnt_off[rid + 1] = n_cnt;
            if (cur_depth > max_ep) max_ep = cur_depth;
            int32_t key;
            if (subtree_level == 2) {
                if (parent_rid == 0) {
                    int32_t second = elen >= 2 ? edge[1] : 255;
                    key = (edge[0] << 8) | second;
                } else {
                    int32_t pk = r->subtree_key[parent_rid];
                    int32_t pf = (pk >> 8) & 0xff, ps = pk & 0xff;
                    key = (ps != 255) ? pk : ((pf << 8) | edge[0]);
                }
            } else {
                key = parent_rid == 0 ? rid : r->subtree_key[parent_rid];
            }
            r->subtree_key[rid] = key;
            if (ec >= 2) {
                if (ftail + 1 > fcap) { fcap *= 2; fr = (int32_t *)realloc(fr, fcap * 3 * 4); }
                fr[ftail * 3] = rid; fr[ftail * 3 + 1] = cur; fr[ftail * 3 + 2] = cur_depth + 1; ftail++;
            }
        }
    }
    free(fr); free(edge);
    r->radix_count = next_id; r->total_edge_chars = n_edge; r->n_depth_files = max_ep + 1;

    /* char positions in depth-file order, then ancestor chains
       (src/cuda/agpt_train.cu:809-846, :892-939) */
    int32_t R = r->radix_count;
    r->edge_start = (int32_t *)calloc((size_t)R, 4);
    int64_t fill = 0;
    for (int32_t d = 0; d < r->n_depth_files; d++)
        for (int32_t i = 1; i < R; i++)
            if (r->endpoint_depth[i] == d) { r->edge_start[i] = (int32_t)fill; fill += r->edge_len[i]; }
    r->anc_off = (int64_t *)malloc((size_t)(R + 1) * 8);
    int64_t *alen = (int64_t *)calloc((size_t)R, 8);
    for (int32_t i = 1; i < R; i++) { int32_t p = r->parent[i]; alen[i] = alen[p] + r->edge_len[p]; }
    r->anc_off[0] = 0;
    for (int32_t i = 0; i < R; i++) r->anc_off[i + 1] = r->anc_off[i] + alen[i];
    r->anc_ids = (int32_t *)malloc((size_t)(r->anc_off[R] ? r->anc_off[R] : 1) * 4);
    for (int32_t i = 1; i < R; i++) {
        int32_t p = r->parent[i];
        int64_t out = r->anc_off[i];
        memcpy(r->anc_ids + out, r->anc_ids + r->anc_off[p], (size_t)alen[p] * 4);
        for (int32_t e = 0; e < r->edge_len[p]; e++) r->anc_ids[out + alen[p] + e] = r->edge_start[p] + e;
    }
    free(alen);
    return r;
}

ORC_API void orc_radix_free(orc_radix *r) {
    if (!r) return;
    free(r->parent); free(r->first_char_depth); free(r->edge_len); free(r->edge_mass);
    free(r->endpoint_depth); free(r->subtree_key); free(r->endpoint_leveled_id);
    free(r->edge_off); free(r->edge_tok);
    free(r->cnt_off); free(r->cnt_tok); free(r->cnt_val);
    free(r->edge_start); free(r->anc_off); free(r->anc_ids);
    free(r);
}

/* Radix directory writer: meta.bin + radix_depth_NNN.bin, byte format of
   src/agpt/streaming_radix_builder.cr:245-256, :291-309, :388-451. */
static void w32(FILE *f, int32_t v) { fwrite(&v, 4, 1, f); }
static void wu32(FILE *f, uint32_t v) { fwrite(&v, 4, 1, f); }
static void w64(FILE *f, int64_t v) { fwrite(&v, 8, 1, f); }

ORC_API int orc_radix_write_dir(const orc_radix *r, const char *dir, int32_t corpus_tokens,
                                int32_t vocab, uint64_t corpus_hash, const char *tag) {
    char path[2048];
    const uint32_t MAGIC = 0x52445841u;
    for (int32_t d = 0; d < r->n_depth_files; d++) {
        snprintf(path, sizeof(path), "%s/radix_depth_%03d.bin", dir, d);
        FILE *f = fopen(path, "wb");
        if (!f) return -1;
        int32_t cnt = 0;
        for (int32_t i = 1; i < r->radix_count; i++) cnt += r->endpoint_depth[i] == d;
        wu32(f, MAGIC); w32(f, d); w32(f, cnt);
        for (int32_t i = 1; i < r->radix_count; i++) {
            if (r->endpoint_depth[i] != d) continue;
            w32(f, i); w32(f, r->parent[i]); w32(f, r->first_char_depth[i]); w32(f, r->edge_len[i]);
            fwrite(r->edge_tok + r->edge_off[i], 4, (size_t)r->edge_len[i], f);
            w32(f, r->edge_mass[i]);
            int32_t ec = (int32_t)(r->cnt_off[i + 1] - r->cnt_off[i]);
            w32(f, ec);
            for (int32_t e = 0; e < ec; e++) { w32(f, r->cnt_tok[r->cnt_off[i] + e]); w32(f, r->cnt_val[r->cnt_off[i] + e]); }
        }
        fclose(f);
    }
    snprintf(path, sizeof(path), "%s/meta.bin", dir);
    FILE *f = fopen(path, "wb");
    if (!f) return -1;
    wu32(f, MAGIC); w32(f, 2); w32(f, r->radix_count); w32(f, r->n_depth_files);
    w64(f, r->total_edge_chars); w32(f, corpus_tokens); w32(f, vocab);
    fwrite(&corpus_hash, 8, 1, f);
    int32_t tl = (int32_t)strlen(tag); w32(f, tl); fwrite(tag, 1, (size_t)tl, f);
    fclose(f);
    return 0;
}

/* ------------------------------------------------------------------------- */
/* RoPE (src/cuda/agpt_train.cu:2298-2321 table; :1305-1351 apply/inverse)   */
/* ------------------------------------------------------------------------- */
ORC_API void orc_rope_table(float *cosv, float *sinv, int max_seq, int dim, float base) {
    int half = dim / 2;
    for (int pos = 0; pos < max_seq; pos++)
        for (int i = 0; i < half; i++) {
            float theta = pos / powf(base, 2.0f * i / dim);
            float c = cosf(theta), s = sinf(theta);
            cosv[pos * dim + 2 * i] = c; cosv[pos * dim + 2 * i + 1] = c;
            sinv[pos * dim + 2 * i] = s; sinv[pos * dim + 2 * i + 1] = s;
        }
}

/* x: [rows, dim] (one row per (node, head)), positions: [rows] */
ORC_API void orc_rope_apply(float *x, const int32_t *pos, const float *cosv, const float *sinv,
                            int64_t rows, int dim, int inverse) {
    for (int64_t r = 0; r < rows; r++) {
        int p = pos[r];
        for (int i = 0; i < dim / 2; i++) {
            float c = cosv[p * dim + 2 * i], s = sinv[p * dim + 2 * i];
            float x0 = x[r * dim + 2 * i], x1 = x[r * dim + 2 * i + 1];
            if (!inverse) { x[r * dim + 2 * i] = x0 * c - x1 * s; x[r * dim + 2 * i + 1] = x0 * s + x1 * c; }
            else          { x[r * dim + 2 * i] = x0 * c + x1 * s; x[r * dim + 2 * i + 1] = -x0 * s + x1 * c; }
        }
    }
}

/* ------------------------------------------------------------------------- */
/* Attention forward on a tree                                               */
/* ------------------------------------------------------------------------- */
static int chain_of(const int32_t *parent, int32_t i, int32_t *buf, int cap) {
    /* fills buf with root-side-first ancestor ids followed by i itself; returns length */
    int len = 0;
    for (int32_t c = i; c >= 0; c = parent[c]) { if (len >= cap) return -1; buf[len++] = c; }
    for (int a = 0, b = len - 1; a < b; a++, b--) { int32_t t = buf[a]; buf[a] = buf[b]; buf[b] = t; }
    return len;
}

static void softmax_row(float *s, int n) {
    float mx = s[0];
    for (int j = 1; j < n; j++) if (s[j] > mx) mx = s[j];
    float sum = 0.f;
    for (int j = 0; j < n; j++) { s[j] = expf(s[j] - mx); sum += s[j]; }
    for (int j = 0; j < n; j++) s[j] /= sum;
}

/* Per-node attention (src/agpt/batched_depth_forward.cr:973-1023).
   w_off[i] (int64) = start of node i's weights; node i stores H rows of depth(i) weights:
   weights[w_off[i] + h*len + p].  Pass weights == NULL to skip saving. */
ORC_API int orc_attn_fwd_per_node(int32_t n, const int32_t *parent, int H, int hd,
                                  const float *q, const float *k, const float *v,
                                  float *out, float *weights, const int64_t *w_off, int max_depth) {
    int D = H * hd;
    float scale = (float)(1.0 / sqrt((double)hd));
    int bad = 0;
#pragma omp parallel
    {
        int32_t *chain = (int32_t *)malloc((size_t)(max_depth + 1) * 4);
        float *s = (float *)malloc((size_t)(max_depth + 1) * 4);
#pragma omp for schedule(dynamic, 256)
        for (int32_t i = 0; i < n; i++) {
            int len = chain_of(parent, i, chain, max_depth + 1);
            if (len < 0) { bad = 1; continue; }
            for (int h = 0; h < H; h++) {
                const float *qh = q + (int64_t)i * D + h * hd;
                for (int p = 0; p < len; p++) {
                    const float *kr = k + (int64_t)chain[p] * D + h * hd;
                    float dot = 0.f;
                    for (int j = 0; j < hd; j++) dot += qh[j] * kr[j];
                    s[p] = dot * scale;
                }
                softmax_row(s, len);
                float *o = out + (int64_t)i * D + h * hd;
                for (int j = 0; j < hd; j++) o[j] = 0.f;
                for (int p = 0; p < len; p++) {
                    const float *vr = v + (int64_t)chain[p] * D + h * hd;
                    for (int j = 0; j < hd; j++) o[j] += s[p] * vr[j];
                }
                if (weights) memcpy(weights + w_off[i] + (int64_t)h * len, s, (size_t)len * 4);
            }
        }
        free(chain); free(s);
    }
    return bad ? -1 : 0;
}

/* Sibling-grouped attention (src/agpt/batched_depth_forward.cr:836-971): the prefix
   scores of a group are one [C, p] product against the parent's chain; the self score
   is per child; out = W[:, :p] V_prefix + w_self v_self.  group_off/group_nodes list the
   children of each parent (all children of one parent in one group). */
ORC_API int orc_attn_fwd_grouped(int32_t n, const int32_t *parent, int32_t n_groups,
                                 const int32_t *group_off, const int32_t *group_nodes,
                                 int H, int hd, const float *q, const float *k, const float *v,
                                 float *out, float *weights, const int64_t *w_off, int max_depth) {
    (void)n;
    int D = H * hd;
    float scale = (float)(1.0 / sqrt((double)hd));
    int bad = 0;
#pragma omp parallel
    {
        int32_t *chain = (int32_t *)malloc((size_t)(max_depth + 1) * 4);
        float *s = (float *)malloc((size_t)(max_depth + 1) * 4);
        float *op = (float *)malloc((size_t)hd * 4);
#pragma omp for schedule(dynamic, 64)
        for (int32_t g = 0; g < n_groups; g++) {
            int32_t first = group_nodes[group_off[g]];
            int32_t par = parent[first];
            int p_len = 0;
            if (par >= 0) { p_len = chain_of(parent, par, chain, max_depth + 1); if (p_len < 0) { bad = 1; continue; } }
            for (int32_t ci = group_off[g]; ci < group_off[g + 1]; ci++) {
                int32_t i = group_nodes[ci];
                for (int h = 0; h < H; h++) {
                    const float *qh = q + (int64_t)i * D + h * hd;
                    for (int p = 0; p < p_len; p++) {
                        const float *kr = k + (int64_t)chain[p] * D + h * hd;
                        float dot = 0.f;
                        for (int j = 0; j < hd; j++) dot += qh[j] * kr[j];
                        s[p] = dot * scale;
                    }
                    const float *ks = k + (int64_t)i * D + h * hd;
                    float dot = 0.f;
                    for (int j = 0; j < hd; j++) dot += qh[j] * ks[j];
                    s[p_len] = dot * scale;
                    softmax_row(s, p_len + 1);
                    for (int j = 0; j < hd; j++) op[j] = 0.f;
                    for (int p = 0; p < p_len; p++) {
                        const float *vr = v + (int64_t)chain[p] * D + h * hd;
                        for (int j = 0; j < hd; j++) op[j] += s[p] * vr[j];
                    }
                    const float *vs = v + (int64_t)i * D + h * hd;
                    float *o = out + (int64_t)i * D + h * hd;
                    for (int j = 0; j < hd; j++) o[j] = op[j] + s[p_len] * vs[j];
                    if (weights) memcpy(weights + w_off[i] + (int64_t)h * (p_len + 1), s, (size_t)(p_len + 1) * 4);
                }
            }
        }
        free(chain); free(s); free(op);
    }
    return bad ? -1 : 0;
}

/* ------------------------------------------------------------------------- */
/* Attention backward (src/agpt/batched_depth_backward.cr:605-695)           */
/*                                                                           */
/* Nodes are visited deepest-first (descending id; parent[i] < i), so a       */
/* node's accumulator already holds every descendant's contribution when the  */
/* node is reached: dk_cur = ds_last*q + accum, dv_cur = w_last*dO + accum.    */
/* Gradients are in post-RoPE space; the caller applies the inverse rotation. */
/* With accumulate_ancestors == 0 the ancestor rows are dropped (the          */
/* local-depth behaviour of src/agpt/trie_walk_trainer.cr:189); with 2 only   */
/* the ancestors on the node's own radix edge are kept, edge_id[a] ==         */
/* edge_id[i] (the CUDA trainer extracts the own-edge part of the packed      */
/* dK/dV and drops the ancestor part, src/cuda/agpt_train.cu:5016-5020).      */
/* ------------------------------------------------------------------------- */
static int attn_bwd_range(int32_t lo, int32_t hi, int h0, int h1, const int32_t *parent, int H, int hd,
                          const float *q, const float *k, const float *v,
                          const float *weights, const int64_t *w_off, const float *d_out,
                          float *dq, float *dk, float *dv, int max_depth, int accumulate_ancestors,
                          const int32_t *edge_id) {
    int D = H * hd;
    float scale = (float)(1.0 / sqrt((double)hd));
    int32_t *chain = (int32_t *)malloc((size_t)(max_depth + 1) * 4);
    float *dw = (float *)malloc((size_t)(max_depth + 1) * 4);
    float *ds = (float *)malloc((size_t)(max_depth + 1) * 4);
    int rc = 0;
    for (int32_t i = hi - 1; i >= lo && rc == 0; i--) {
        int len = chain_of(parent, i, chain, max_depth + 1);
        if (len < 0) { rc = -1; break; }
        for (int h = h0; h < h1; h++) {
            const float *w = weights + w_off[i] + (int64_t)h * len;
            const float *qh = q + (int64_t)i * D + h * hd;
            const float *go = d_out + (int64_t)i * D + h * hd;
            double dot = 0.0;
            for (int p = 0; p < len; p++) {
                const float *vr = v + (int64_t)chain[p] * D + h * hd;
                float sum = 0.f;
                for (int j = 0; j < hd; j++) sum += go[j] * vr[j];
                dw[p] = sum;
                dot += (double)sum * (double)w[p];
            }
            for (int p = 0; p < len; p++) ds[p] = (float)((double)w[p] * ((double)dw[p] - dot) * (double)scale);
            float *dqh = dq + (int64_t)i * D + h * hd;
            for (int j = 0; j < hd; j++) {
                float sum = 0.f;
                for (int p = 0; p < len; p++) sum += ds[p] * k[(int64_t)chain[p] * D + h * hd + j];
                dqh[j] = sum;
            }
            for (int p = 0; p < len; p++) {
                if (p == len - 1) {
                    float *dkc = dk + (int64_t)i * D + h * hd, *dvc = dv + (int64_t)i * D + h * hd;
                    for (int j = 0; j < hd; j++) {
                        dkc[j] = ds[p] * qh[j] + dkc[j];
                        dvc[j] = w[p] * go[j] + dvc[j];
                    }
                } else if (accumulate_ancestors == 1 || (accumulate_ancestors == 2 && edge_id[chain[p]] == edge_id[i])) {
                    float *dka = dk + (int64_t)chain[p] * D + h * hd, *dva = dv + (int64_t)chain[p] * D + h * hd;
                    for (int j = 0; j < hd; j++) { dka[j] += ds[p] * qh[j]; dva[j] += w[p] * go[j]; }
                }
            }
        }
    }
    free(chain); free(dw); free(ds);
    return rc;
}

/* unit_off: [n_units+1] id ranges that are closed under "ancestor of" (root-child
   subtrees of an id order in which each subtree is contiguous); NULL = one unit.  Units
   and heads are independent, so (unit, head) pairs run in parallel without changing any
   per-element summation order. */
ORC_API int orc_attn_bwd(int32_t n, const int32_t *parent, int H, int hd,
                         const float *q, const float *k, const float *v,
                         const float *weights, const int64_t *w_off, const float *d_out,
                         float *dq, float *dk, float *dv, int max_depth, int accumulate_ancestors,
                         int32_t n_units, const int32_t *unit_off, const int32_t *edge_id) {
    int D = H * hd;
    memset(dk, 0, (size_t)n * D * 4);      /* dk/dv double as the per-node accumulators */
    memset(dv, 0, (size_t)n * D * 4);
    int32_t one[2] = {0, n};
    if (!unit_off) { unit_off = one; n_units = 1; }
    if (accumulate_ancestors == 2 && !edge_id) return -1;
    int bad = 0;
    int64_t n_tasks = (int64_t)n_units * H;
#pragma omp parallel for schedule(dynamic, 1)
    for (int64_t t = 0; t < n_tasks; t++) {
        int32_t u = (int32_t)(t / H); int h = (int)(t % H);
        if (attn_bwd_range(unit_off[u], unit_off[u + 1], h, h + 1, parent, H, hd, q, k, v, weights, w_off,
                           d_out, dq, dk, dv, max_depth, accumulate_ancestors, edge_id) != 0) bad = 1;
    }
    return bad ? -1 : 0;
}

/* Matrix form of one (node, head) backward, as the reference spec states it
   (spec/agpt_backward_attention_spec.cr:185-276).  K, V: [len, hd] rows of the chain;
   w, d_out, qv as above; accum_dk/accum_dv: the node's own accumulator (added at the
   last row).  Outputs dk_full/dv_full [len, hd] and dq [hd]. */
ORC_API void orc_attn_bwd_head_matrix(int len, int hd, const float *K, const float *V,
                                      const float *w, const float *qv, const float *go,
                                      const float *accum_dk, const float *accum_dv,
                                      float *dq, float *dk_full, float *dv_full) {
    float scale = (float)(1.0 / sqrt((double)hd));
    float *dwv = (float *)malloc((size_t)len * 4), *dsv = (float *)malloc((size_t)len * 4);
    for (int p = 0; p < len; p++)
        for (int j = 0; j < hd; j++) dv_full[p * hd + j] = w[p] * go[j];           /* w^T dO */
    for (int p = 0; p < len; p++) {
        float s = 0.f;
        for (int j = 0; j < hd; j++) s += go[j] * V[p * hd + j];                  /* dO V^T */
        dwv[p] = s;
    }
    double dot = 0.0;
    for (int p = 0; p < len; p++) dot += (double)dwv[p] * (double)w[p];
    for (int p = 0; p < len; p++) dsv[p] = (float)((double)w[p] * ((double)dwv[p] - dot));
    for (int p = 0; p < len; p++) dsv[p] *= scale;
    for (int j = 0; j < hd; j++) {
        float s = 0.f;
        for (int p = 0; p < len; p++) s += dsv[p] * K[p * hd + j];
        dq[j] = s;
    }
    for (int p = 0; p < len; p++)
        for (int j = 0; j < hd; j++) dk_full[p * hd + j] = dsv[p] * qv[j];
    for (int j = 0; j < hd; j++) {
        dk_full[(len - 1) * hd + j] += accum_dk[j];
        dv_full[(len - 1) * hd + j] += accum_dv[j];
    }
    free(dwv); free(dsv);
}

/* One (node, head) of the optimized routine with explicit accumulators, for the
   formula-equivalence known-answer test (src/agpt/batched_depth_backward.cr:628-690).
   anc_dk/anc_dv: [len-1, hd] ancestor accumulators, updated in place. */
ORC_API void orc_attn_bwd_head_optimized(int len, int hd, const float *K, const float *V,
                                         const float *w, const float *qv, const float *go,
                                         const float *accum_dk, const float *accum_dv,
                                         float *dq, float *dk_cur, float *dv_cur,
                                         float *anc_dk, float *anc_dv) {
    float scale = (float)(1.0 / sqrt((double)hd));
    float *dwv = (float *)malloc((size_t)len * 4), *dsv = (float *)malloc((size_t)len * 4);
    double dot = 0.0;
    for (int p = 0; p < len; p++) {
        float sum = 0.f;
        for (int j = 0; j < hd; j++) sum += go[j] * V[p * hd + j];
        dwv[p] = sum; dot += (double)sum * (double)w[p];
    }
    for (int p = 0; p < len; p++) dsv[p] = (float)((double)w[p] * ((double)dwv[p] - dot) * (double)scale);
    for (int j = 0; j < hd; j++) {
        float sum = 0.f;
        for (int p = 0; p < len; p++) sum += dsv[p] * K[p * hd + j];
        dq[j] = sum;
    }
    for (int p = 0; p < len; p++) {
        if (p == len - 1) {
            for (int j = 0; j < hd; j++) { dk_cur[j] = dsv[p] * qv[j] + accum_dk[j]; dv_cur[j] = w[p] * go[j] + accum_dv[j]; }
        } else {
            for (int j = 0; j < hd; j++) { anc_dk[p * hd + j] += dsv[p] * qv[j]; anc_dv[p * hd + j] += w[p] * go[j]; }
        }
    }
    free(dwv); free(dsv);
}

/* ------------------------------------------------------------------------- */
/* Packed-prefix layout of the legacy kernel boundary                        */
/* (src/agpt/batched_depth_forward.cr:656-801; radix: agpt_train.cu:3106-3117,*/
/* :4445-4483).  Query t belongs to node query_to_node[t]; it attends the     */
/* first kv_lengths[node] - (query_offsets[node+1] - t) + 1 packed rows of    */
/* that node: all ancestors plus own-edge rows 0..j.                          */
/* k/v: [(kv_off + pos) * H + h] * hd.  weights: [(t*H + h) * max_len + pos]. */
/* With query_to_node == NULL every node has exactly one query (leveled form).*/
/* ------------------------------------------------------------------------- */
ORC_API void orc_packed_attn_fwd(const float *q, const float *k, const float *v,
                                 const int32_t *query_to_node, const int32_t *query_offsets,
                                 const int32_t *kv_offsets, const int32_t *kv_lengths,
                                 float *out, float *weights, int T_q, int H, int hd, int max_len,
                                 float scale) {
    float *s = (float *)malloc((size_t)(max_len + 1) * 4);
    for (int t = 0; t < T_q; t++) {
        int node = query_to_node ? query_to_node[t] : t;
        int len = query_to_node ? kv_lengths[node] - (query_offsets[node + 1] - t) + 1 : kv_lengths[node];
        int64_t off = kv_offsets[node];
        for (int h = 0; h < H; h++) {
            const float *qh = q + ((int64_t)t * H + h) * hd;
            for (int p = 0; p < len; p++) {
                const float *kr = k + ((off + p) * H + h) * hd;
                float dot = 0.f;
                for (int j = 0; j < hd; j++) dot += qh[j] * kr[j];
                s[p] = dot * scale;
            }
            softmax_row(s, len);
            float *o = out + ((int64_t)t * H + h) * hd;
            for (int j = 0; j < hd; j++) o[j] = 0.f;
            for (int p = 0; p < len; p++) {
                const float *vr = v + ((off + p) * H + h) * hd;
                for (int j = 0; j < hd; j++) o[j] += s[p] * vr[j];
            }
            float *wr = weights + ((int64_t)t * H + h) * max_len;
            for (int p = 0; p < max_len; p++) wr[p] = p < len ? s[p] : 0.f;
        }
    }
    free(s);
}

/* dk_full/dv_full are accumulated into (the caller zeroes them), dq is written. */
ORC_API void orc_packed_attn_bwd(const float *q, const float *k, const float *v,
                                 const float *weights, const float *d_out,
                                 const int32_t *query_to_node, const int32_t *query_offsets,
                                 const int32_t *kv_offsets, const int32_t *kv_lengths,
                                 float *dq, float *dk_full, float *dv_full,
                                 int T_q, int H, int hd, int max_len, float scale) {
    float *dw = (float *)malloc((size_t)(max_len + 1) * 4), *ds = (float *)malloc((size_t)(max_len + 1) * 4);
    for (int t = 0; t < T_q; t++) {
        int node = query_to_node ? query_to_node[t] : t;
        int len = query_to_node ? kv_lengths[node] - (query_offsets[node + 1] - t) + 1 : kv_lengths[node];
        int64_t off = kv_offsets[node];
        for (int h = 0; h < H; h++) {
            const float *qh = q + ((int64_t)t * H + h) * hd;
            const float *go = d_out + ((int64_t)t * H + h) * hd;
            const float *w = weights + ((int64_t)t * H + h) * max_len;
            double dot = 0.0;
            for (int p = 0; p < len; p++) {
                const float *vr = v + ((off + p) * H + h) * hd;
                float sum = 0.f;
                for (int j = 0; j < hd; j++) sum += go[j] * vr[j];
                dw[p] = sum; dot += (double)sum * (double)w[p];
            }
            for (int p = 0; p < len; p++) ds[p] = (float)((double)w[p] * ((double)dw[p] - dot) * (double)scale);
            float *dqh = dq + ((int64_t)t * H + h) * hd;
            for (int j = 0; j < hd; j++) {
                float sum = 0.f;
                for (int p = 0; p < len; p++) sum += ds[p] * k[((off + p) * H + h) * hd + j];
                dqh[j] = sum;
            }
            for (int p = 0; p < len; p++) {
                float *dkr = dk_full + ((off + p) * H + h) * hd, *dvr = dv_full + ((off + p) * H + h) * hd;
                for (int j = 0; j < hd; j++) { dkr[j] += ds[p] * qh[j]; dvr[j] += w[p] * go[j]; }
            }
        }
    }
    free(dw); free(ds);
}

/* ------------------------------------------------------------------------- */
/* Loss                                                                      */
/* ------------------------------------------------------------------------- */
static void softmax_probs(const float *in, float *p, int V) {
    float mx = -3.402823466e+38f;
    for (int j = 0; j < V; j++) if (in[j] > mx) mx = in[j];
    float sum = 0.f;
    for (int j = 0; j < V; j++) { p[j] = expf(in[j] - mx); sum += p[j]; }
    float inv = 1.0f / sum;
    for (int j = 0; j < V; j++) p[j] *= inv;
}

/* Per-query loss of the radix trainer (src/cuda/agpt_train.cu:2069-2197). */
ORC_API void orc_loss_per_query(const float *logits, const int32_t *query_to_node,
                                const int32_t *query_offsets, const int32_t *radix_ids,
                                const int32_t *token_ids, const int32_t *counts_offset,
                                const int32_t *counts_tok, const int32_t *counts_val,
                                const float *mass_weights, float *d_logits, float *loss_out,
                                int T_q, int V, float entropy_lambda, float intermediate_weight,
                                int ce_only) {
    for (int q = 0; q < T_q; q++) {
        float *g = d_logits + (int64_t)q * V;
        softmax_probs(logits + (int64_t)q * V, g, V);
        int n_idx = query_to_node[q];
        int is_endpoint = (q + 1) == query_offsets[n_idx + 1];
        int ce_as_intermediate = ce_only && is_endpoint && (q + 1 < T_q);
        if (is_endpoint && !ce_as_intermediate) {
            int rid = radix_ids[n_idx];
            int start = counts_offset[rid], end = counts_offset[rid + 1];
            if (start == end) { loss_out[q] = 0.f; continue; }
            int total = 0;
            for (int e = start; e < end; e++) total += counts_val[e];
            float total_f = (float)total;
            float weight = 1.0f;
            if (entropy_lambda > 0.0f && (end - start) > 1) {
                float Hh = 0.f;
                for (int e = start; e < end; e++) { float qe = counts_val[e] / total_f; if (qe > 0.f) Hh -= qe * logf(qe); }
                weight = 1.0f + entropy_lambda * (Hh / logf((float)V));
            }
            if (mass_weights) weight *= mass_weights[q];
            float loss = 0.f;
            for (int e = start; e < end; e++) {
                int tok = counts_tok[e]; int cnt = counts_val[e];
                loss -= (cnt / total_f) * logf(g[tok] + 1e-10f);
                g[tok] -= cnt / total_f;
            }
            if (weight != 1.0f) { loss *= weight; for (int j = 0; j < V; j++) g[j] *= weight; }
            loss_out[q] = loss;
        } else {
            int target = token_ids[q + 1];
            float loss = -logf(g[target] + 1e-10f);
            g[target] -= 1.0f;
            float w = intermediate_weight;
            if (mass_weights) w *= mass_weights[q];
            if (w != 1.0f) { loss *= w; for (int j = 0; j < V; j++) g[j] *= w; }
            loss_out[q] = loss;
        }
    }
}

/* Per-node loss of the leveled trainer (src/cuda/agpt_train.cu:1947-2029). */
ORC_API void orc_loss_per_node(const float *logits, const int32_t *node_ids,
                               const int32_t *counts_offset, const int32_t *counts_tok,
                               const int32_t *counts_val, float *d_logits, float *loss_out,
                               int N, int V) {
    for (int i = 0; i < N; i++) {
        float *g = d_logits + (int64_t)i * V;
        softmax_probs(logits + (int64_t)i * V, g, V);
        int nid = node_ids[i];
        int start = counts_offset[nid], end = counts_offset[nid + 1];
        if (start == end) { loss_out[i] = 0.f; continue; }
        int total = 0;
        for (int e = start; e < end; e++) total += counts_val[e];
        float total_f = (float)total, loss = 0.f;
        for (int e = start; e < end; e++) {
            int tok = counts_tok[e]; int cnt = counts_val[e];
            loss -= (cnt / total_f) * logf(g[tok] + 1e-10f);
            g[tok] -= cnt / total_f;
        }
        loss_out[i] = loss;
    }
}

/* Per-node count-weighted loss of the Crystal walker, f64 log
   (src/agpt/trie_walk_trainer.cr:118-158).  loss_out is f64 per node; nodes without
   counts get loss 0 and an all-zero gradient row (they are skipped there). */
ORC_API void orc_loss_crystal(const float *logits, const int32_t *counts_offset,
                              const int32_t *counts_tok, const int32_t *counts_val,
                              float *d_logits, double *loss_out, int N, int V, double lambda) {
    float *p = (float *)malloc((size_t)V * 4);
    double log_vocab = log((double)V);
    for (int i = 0; i < N; i++) {
        float *g = d_logits + (int64_t)i * V;
        int start = counts_offset[i], end = counts_offset[i + 1];
        if (start == end) { loss_out[i] = 0.0; memset(g, 0, (size_t)V * 4); continue; }
        softmax_probs(logits + (int64_t)i * V, p, V);
        int total = 0;
        for (int e = start; e < end; e++) total += counts_val[e];
        double total_f = (double)total, entropy = 0.0;
        if (lambda > 0.0 && end - start > 1)
            for (int e = start; e < end; e++) { double qe = counts_val[e] / total_f; if (qe > 0.0) entropy -= qe * log(qe); }
        double weight = lambda > 0.0 ? 1.0 + lambda * (entropy / log_vocab) : 1.0;
        double loss = 0.0;
        for (int e = start; e < end; e++) loss -= counts_val[e] * log((double)p[counts_tok[e]] + 1e-10);
        loss /= total; loss *= weight;
        float wf = (float)weight;
        for (int j = 0; j < V; j++) g[j] = p[j] * wf;
        for (int e = start; e < end; e++) g[counts_tok[e]] -= ((float)counts_val[e] / total) * wf;
        loss_out[i] = loss;
    }
    free(p);
}

/* Chunk mass weights (src/cuda/agpt_train.cu:4608-4637): per radix node
   f(edge_mass) with f in {1: log1p, 2: sqrt, 3: linear}, normalised by the mean over the
   chunk's queries, broadcast to the node's queries. */
ORC_API void orc_mass_weights(const int32_t *edge_mass, const int32_t *edge_len, int N, int mode,
                              float *out_per_query) {
    double total_w = 0.0; int64_t T_q = 0;
    float *nw = (float *)malloc((size_t)(N ? N : 1) * 4);
    for (int i = 0; i < N; i++) {
        float c = (float)edge_mass[i], w;
        switch (mode) { case 1: w = logf(1.0f + c); break; case 2: w = sqrtf(c); break; case 3: w = c; break; default: w = 1.0f; }
        nw[i] = w; total_w += (double)w * edge_len[i]; T_q += edge_len[i];
    }
    float mean_w = T_q > 0 ? (float)(total_w / T_q) : 1.0f;
    if (mean_w <= 0.0f) mean_w = 1.0f;
    int64_t qi = 0;
    for (int i = 0; i < N; i++) { float w = nw[i] / mean_w; for (int j = 0; j < edge_len[i]; j++) out_per_query[qi++] = w; }
    free(nw);
}

/* Layer norm of the reference's CPU path: float32 mean and biased variance, std_inv = 1/sqrt(var + 1e-5)
   (src/agpt/incremental_forward.cr:143-163); backward with float64 row means, dgamma/dbeta accumulated
   (src/agpt/batched_depth_backward.cr:751-799). */
ORC_API void orc_layer_norm_fwd(const float *x, float *y, float *norm, float *std_inv, const float *gamma,
                                const float *beta, int64_t rows, int cols) {
    for (int64_t r = 0; r < rows; r++) {
        const float *xr = x + r * cols;
        float mean = 0.f;
        for (int j = 0; j < cols; j++) mean += xr[j];
        mean /= cols;
        float var = 0.f;
        for (int j = 0; j < cols; j++) { float d = xr[j] - mean; var += d * d; }
        var /= cols;
        float sinv = (float)(1.0 / sqrt((double)(var + 1e-5f)));
        std_inv[r] = sinv;
        for (int j = 0; j < cols; j++) {
            float nrm = (xr[j] - mean) * sinv;
            norm[r * cols + j] = nrm;
            y[r * cols + j] = nrm * gamma[j] + beta[j];
        }
    }
}

ORC_API void orc_layer_norm_bwd(const float *grad, const float *norm, const float *std_inv, const float *gamma,
                                float *dx, float *dgamma, float *dbeta, int64_t rows, int cols) {
    for (int64_t r = 0; r < rows; r++) {
        const float *g = grad + r * cols, *nm = norm + r * cols;
        double sinv = std_inv[r], mean_dn = 0.0, mean_dn_n = 0.0;
        for (int j = 0; j < cols; j++) { dgamma[j] += g[j] * nm[j]; dbeta[j] += g[j]; }
        for (int j = 0; j < cols; j++) { float dn = g[j] * gamma[j]; mean_dn += dn; mean_dn_n += dn * nm[j]; }
        mean_dn /= cols; mean_dn_n /= cols;
        for (int j = 0; j < cols; j++) { float dn = g[j] * gamma[j]; dx[r * cols + j] = (float)((dn - mean_dn - nm[j] * mean_dn_n) * sinv); }
    }
}

ORC_API void orc_set_num_threads(int n) {
#ifdef _OPENMP
    if (n > 0) omp_set_num_threads(n);
#else
    (void)n;
#endif
}

ORC_API int orc_num_threads(void) {
#ifdef _OPENMP
    return omp_get_max_threads();
#else
    return 1;
#endif
}
