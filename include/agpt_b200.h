/*
 * agpt_b200.h — C ABI of libagpt_b200.so: the trie-walk attention hot path of AGPT
 * (forward, backward, mass-weighted next-token loss, per-subtree KV store and walker
 * index) written for NVIDIA B200 (sm_100a).
 *
 * Two groups of entry points:
 *
 *  1. The legacy kernel boundary: the symbols the reference's Crystal `lib
 *     LibCUDAKernels` binding and its C++ trainer link against, with identical names,
 *     argument order and packed-prefix buffer layout.  Citations are to files of the
 *     reference project.
 *  2. The native tree-indexed boundary (`agpt_b200_*`): the same maths addressed through
 *     a walker plan (depth-first node order, subtree intervals, per-tile ancestor chains)
 *     instead of materialised per-node prefixes.
 *
 * Conventions: all pointers named `d_*` or documented as device pointers are CUDA device
 * memory owned by the caller; the library never retains them.  `int` status returns are
 * 0 on success and a negative AGPT_E_* code otherwise; agpt_b200_last_error() gives the
 * message of the calling thread's last failure.  No function traps or aborts.
 */
#ifndef AGPT_B200_H
#define AGPT_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define AGPT_OK 0
#define AGPT_E_ARG (-1)      /* bad argument (null pointer, unsupported head_dim, ...) */
#define AGPT_E_CUDA (-2)     /* a CUDA runtime call or kernel launch failed */
#define AGPT_E_IO (-3)       /* file could not be read or written, or has a bad magic */
#define AGPT_E_LIMIT (-4)    /* size beyond a documented maximum */
#define AGPT_E_NOMEM (-5)

#define AGPT_KV_F32 0
#define AGPT_KV_BF16 1

const char *agpt_b200_last_error(void);
const char *agpt_b200_version(void);

/* ======================================================================== */
/* 1. Legacy kernel boundary                                                */
/* ======================================================================== */

/* Replaces cuda_batched_varlen_attention (declared src/cuda/agpt_train.cu:73-77; called
 * src/agpt/batched_depth_forward.cr:767-771 and src/cuda/agpt_train.cu:2805-2809).
 * q_packed [n_nodes*n_heads, head_dim]; k/v_packed [(kv_offsets[i]+pos)*n_heads+h]*head_dim;
 * output [n_nodes*n_heads, head_dim]; weights_out [(i*n_heads+h)*max_len + pos]. */
void cuda_batched_varlen_attention(const float *q_packed, const float *k_packed, const float *v_packed,
                                   const int *kv_offsets, const int *kv_lengths, float *output,
                                   float *weights_out, int n_nodes, int n_heads, int head_dim, int max_len,
                                   float scale);

/* Replaces cuda_batched_varlen_attention_backward (declared src/cuda/agpt_train.cu:78-83;
 * called src/agpt/batched_depth_backward.cr:471-476, src/cuda/agpt_train.cu:2997-3002).
 * dq [n_nodes*n_heads, head_dim]; dk_full/dv_full in the packed-prefix layout, fully written. */
void cuda_batched_varlen_attention_backward(const float *q_packed, const float *k_packed,
                                            const float *v_packed, const float *attn_weights,
                                            const float *d_out, const int *kv_offsets, const int *kv_lengths,
                                            float *dq, float *dk_full, float *dv_full, int n_nodes,
                                            int n_heads, int head_dim, int max_len, float scale);

/* Replaces cuda_unpack_batched_attn_output (declared src/cuda/agpt_train.cu:84-86; called
 * src/agpt/batched_depth_forward.cr:776-778): [n*H, hd] -> [n, H*hd]. */
void cuda_unpack_batched_attn_output(const float *packed_output, float *unpacked_output, int n_nodes,
                                     int n_heads, int head_dim);

/* Replaces cuda_batched_varlen_attention_L_queries (declared src/cuda/agpt_train.cu:3120-3125;
 * called :4740-4744): query t of radix node query_to_node[t] attends the node's ancestors plus its
 * own edge rows 0..j, i.e. the first kv_lengths[node] - (query_offsets[node+1] - t) + 1 packed rows. */
void cuda_batched_varlen_attention_L_queries(const float *q_packed, const float *k_packed,
                                             const float *v_packed, const int *query_to_node,
                                             const int *query_offsets, const int *kv_offsets,
                                             const int *kv_lengths, float *output, float *weights_out,
                                             int T_q, int n_heads, int head_dim, int max_kv_len, float scale);

/* Replaces cuda_batched_varlen_attention_L_queries_backward (declared
 * src/cuda/agpt_train.cu:3126-3132; called :4988-4992).  dk_full/dv_full are accumulated into and
 * must be zeroed by the caller (:4983-4984); the accumulation order is fixed (no atomics). */
void cuda_batched_varlen_attention_L_queries_backward(const float *q_packed, const float *k_packed,
                                                      const float *v_packed, const float *attn_weights,
                                                      const float *d_out, const int *query_to_node,
                                                      const int *query_offsets, const int *kv_offsets,
                                                      const int *kv_lengths, float *dq, float *dk_full,
                                                      float *dv_full, int T_q, int n_heads, int head_dim,
                                                      int max_kv_len, float scale);

/* Replaces cuda_sync (declared src/cuda/agpt_train.cu:87; called
 * src/agpt/batched_depth_forward.cr:772): cudaDeviceSynchronize. */
void cuda_sync(void);

/* ======================================================================== */
/* 2. Native boundary                                                        */
/* ======================================================================== */

/* ---- synthetic workloads (seeded; stand-ins for the reference's corpora) ---- */

/* Order-`order` Markov chain over `vocab` symbols with Zipf(1.1) unigram marginals. */
int agpt_b200_synth_markov_corpus(int64_t n, int vocab, int order, uint64_t seed, int32_t *out);
/* The same source with long verbatim repeats injected: before each symbol one more draw of the same splitmix64
 * stream decides, with probability 2^-repeat_log2, to copy a span of 64 + (draw mod 193) symbols starting at a
 * uniformly drawn earlier offset.  Stand-in for the deep repeats of natural text: the count>=2 trie of a plain
 * order-4 Markov source ends near depth 24, with repeats it reaches the depth cap. */
int agpt_b200_synth_markov_corpus_repeats(int64_t n, int vocab, int order, uint64_t seed, int repeat_log2,
                                          int32_t *out);

/* Level-capped random tree in breadth-first id order; parent_out[i] == -1 for the root's
 * children.  Returns the node count (<= max_nodes) or a negative error. */
int64_t agpt_b200_synth_tree(int64_t max_nodes, int max_depth, int root_children, double p_stop,
                             int max_children, int64_t level_cap, uint64_t seed, int32_t *parent_out);

/* Per-query mass weights of one launch: w = f(edge_mass) / mean over the counted queries, f = 1, log(1 + m), sqrt(m)
 * or m for mode 0..3 (off, log, sqrt, linear) -- the host loop of src/cuda/agpt_train.cu:4608-4637 with the mean taken
 * inside each unit (unit_of_node, NULL = one unit), so that weights do not depend on how units are packed into
 * launches.  One entry per loss node; a node with counted[i] == 0 (a context row) gets a weight but does not enter
 * the mean (counted NULL = all counted).  out_per_query holds sum(edge_len) floats, node by node. */
int agpt_b200_mass_weights(const int32_t *edge_mass, const int32_t *edge_len, const int32_t *unit_of_node,
                           const uint8_t *counted, int64_t n_nodes, int64_t n_units, int mode, float *out_per_query);

/* ---- radix trie: build, on-disk directory format, char-position tree ---- */

typedef struct agpt_trie agpt_trie;

typedef struct {
    int32_t radix_count;        /* including the virtual root, id 0 */
    int32_t n_depth_files;      /* max endpoint depth + 1 */
    int64_t total_edge_chars;   /* number of char positions (= attention queries per layer) */
    int64_t total_counts;
    int64_t leveled_nodes;      /* nodes of the depth-capped trie incl. root; 0 if loaded from disk */
    const int32_t *parent, *first_char_depth, *edge_len, *edge_mass, *endpoint_depth, *subtree_key;
    const int64_t *edge_off;    /* [radix_count+1] into edge_tok (emission order) */
    const int32_t *edge_tok;
    const int64_t *cnt_off;     /* [radix_count+1] */
    const int32_t *cnt_tok, *cnt_val;
    const int32_t *edge_start;  /* char position of the first edge char (file order) */
} agpt_trie_info;

/* Replaces StreamingLeveledBuilder#build + StreamingRadixBuilder#build
 * (src/agpt/streaming_leveled_builder.cr:31, src/agpt/streaming_radix_builder.cr:103): same node
 * numbering, counts, edge_mass, pruning rule and subtree keys. */
int agpt_b200_trie_build(const int32_t *corpus, int64_t n, int max_depth, int subtree_level,
                         int prune_min_mass, int prune_min_depth, agpt_trie **out);
/* Replaces load_radix_trie (src/cuda/agpt_train.cu:772-946): reads meta.bin + radix_depth_NNN.bin. */
int agpt_b200_trie_load_dir(const char *dir, agpt_trie **out);
/* Writes meta.bin, radix_depth_NNN.bin and, when per_subtree != 0, subtrees/radix_subtree_KKKKKK.bin
 * + manifest.bin, byte-identical to src/agpt/streaming_radix_builder.cr:245-343, :388-451. */
int agpt_b200_trie_save_dir(const agpt_trie *t, const char *dir, int per_subtree, int32_t corpus_tokens,
                            int32_t vocab, uint64_t corpus_hash, const char *tokenizer_tag);
/* Replaces load_manifest and load_subtree (src/cuda/agpt_train.cu:431-493, :495-669): manifest.bin lists the
 * per-subtree files (key, radix nodes, edge chars, deepest endpoint; returns their number, fills at most cap entries);
 * a subtree file becomes a trie of its own with local ids (0 = root, records 1..n in file order, char positions in
 * file order); a parent that is the virtual root or is not in the file (the depth-1 node above a bigram subtree)
 * becomes the local root. */
int64_t agpt_b200_trie_manifest(const char *dir, int64_t cap, int32_t *keys, int32_t *n_nodes, int64_t *edge_chars,
                                int32_t *max_endpoint_depth);
int agpt_b200_trie_load_subtree(const char *dir, int32_t subtree_key, agpt_trie **out);
int agpt_b200_trie_info(const agpt_trie *t, agpt_trie_info *out);
/* The same trie (identical arrays, node for node) built from a suffix order: sa[0 .. n-2] are the start positions
 * 0 .. n-2 ordered by their first max_depth + 1 tokens (a position past the end of the corpus orders before every
 * token), lcp[i] the number of equal leading tokens of sa[i-1] and sa[i] within those max_depth + 1 (lcp[0] = 0).
 * agpt_b200_suffix_order_gpu computes both on the device (one stable radix pass per token of the key, then one
 * thread per neighbouring pair; device_ms_out, if not NULL, receives the device time); agpt_b200_trie_build_gpu
 * chains the two.  They replace the bucket refinement of the level-by-level build
 * (src/agpt/streaming_leveled_builder.cr:31-118) and the breadth-first compression
 * (src/agpt/streaming_radix_builder.cr:103-343) by a sort and a linear pass.  n must be at least max_depth + 2. */
int agpt_b200_trie_from_suffix_order(const int32_t *corpus, int64_t n, int max_depth, int subtree_level,
                                     int prune_min_mass, int prune_min_depth, const int32_t *sa, const int32_t *lcp,
                                     agpt_trie **out);
int agpt_b200_suffix_order_gpu(const int32_t *corpus, int64_t n, int key_len, int device, int32_t *sa_out,
                               int32_t *lcp_out, float *device_ms_out);
int agpt_b200_trie_build_gpu(const int32_t *corpus, int64_t n, int max_depth, int subtree_level, int prune_min_mass,
                             int prune_min_depth, int device, agpt_trie **out);
/* Stochastic training units of the reference's "lightning" mode (src/cuda/agpt_train.cu:152-200, :4060-4241): `steps`
 * samples from a 32-bit xorshift generator (*rng_state, the reference seeds it with 0x5c115e1).  sampler 1: uniform
 * over radix nodes; 2: uniform over root children; 3: mass-weighted walk from the root that stops with probability
 * p_stop at each level (forced on while the node's mass exceeds max_mass > 0); 4: the same walk down to a leaf.  A
 * sample's node set is its ancestors (n_anc_out of them: context only), the sampled node and its descendants
 * breadth first (sampler 4: the root-to-node path), stably ordered by endpoint depth; mass_out is the summed edge
 * mass.  Returns the total number of node ids; with nodes_out == NULL nothing is written and the generator state is
 * left as it was (call once to size nodes_out, once to fill). */
int64_t agpt_b200_lightning_sample(const agpt_trie *t, int sampler, int steps, float p_stop, int64_t max_mass,
                                   uint32_t *rng_state, int32_t *sample_out, int32_t *n_anc_out, int64_t *node_off_out,
                                   double *mass_out, int32_t *nodes_out, int64_t nodes_cap);
/* Learning rate of optimizer step number `step` (steps already taken) out of total_steps: schedule 0 constant,
 * 1 cosine decay, 2 linear warm-up over warmup_steps then cosine decay (src/cuda/agpt_train.cu:146-216), float32. */
float agpt_b200_compute_lr(float base_lr, int step, int total_steps, int warmup_steps, int schedule);
void agpt_b200_trie_free(agpt_trie *t);
/* FNV-1a corpus hash (src/agpt/trie_corpus.cr:120-134). */
uint64_t agpt_b200_token_hash(const int32_t *tokens, int64_t n);

/* Char-position tree of a radix trie, in the trainer's char numbering
 * (src/cuda/agpt_train.cu:832, :892-939): parent char (-1 under the root), token, absolute depth
 * (1-based), owning radix id.  Each output array has total_edge_chars entries; any may be NULL. */
int agpt_b200_trie_char_tree(const agpt_trie *t, int32_t *parent, int32_t *token, int32_t *depth,
                             int32_t *radix_of_char);

/* ---- walker plan: depth-first layout of a tree + tile index ---- */

typedef struct agpt_plan agpt_plan;

typedef struct {
    int64_t n;                  /* nodes */
    int32_t tile_m;             /* queries per tile */
    int64_t n_tiles;
    int64_t chain_rows;         /* sum over tiles of the first query's ancestor count */
    int32_t max_depth;
    int64_t sum_depth;          /* sum over nodes of depth (attended rows incl. self) */
    int64_t sum_group_prefix;   /* sum over sibling groups of the shared prefix length */
    int64_t n_groups;           /* sibling groups */
    int64_t n_reduce_items, n_reduce_nodes, n_reduce_multi;   /* dK/dV reduction work list sizes */
    const int32_t *dfs_to_node; /* host: node id at each depth-first position */
    const int32_t *node_to_dfs; /* host */
    const int32_t *parent_dfs;  /* host: parent position (-1 under the root) */
    const int32_t *depth;       /* host: 1-based */
    const int32_t *sub_end;     /* host: one past the last position of the node's subtree */
    int device;                 /* CUDA device holding the index arrays, -1 = none */
} agpt_plan_info;

/* Replaces the ancestor index (src/agpt/batched_depth_forward.cr:351-359,
 * src/cuda/agpt_train.cu:892-939, :1126-1198) and the walker's ordering
 * (src/cuda/agpt_train.cu:3602-3736).  parent[i] is a node id or -1; any id order is accepted.
 * With device >= 0 the index arrays are also allocated on that device (freed by plan_destroy). */
int agpt_b200_plan_create(const int32_t *parent, int64_t n, int tile_m, int device, agpt_plan **out);
int agpt_b200_plan_info(const agpt_plan *p, agpt_plan_info *out);
void agpt_b200_plan_destroy(agpt_plan *p);
/* Bytes of scratch attn_bwd needs for `d_model` columns. */
int64_t agpt_b200_attn_bwd_workspace_bytes(const agpt_plan *p, int d_model);

/* Root-child / bigram units of a plan as depth-first ranges (src/cuda/agpt_train.cu:3602-3623,
 * src/agpt/streaming_radix_builder.cr:215-240).  level 1: one unit per depth-1 node; level 2: one
 * per depth-2 node, the depth-1 node itself forming a unit of one.  Writes up to cap ranges into
 * unit_begin/unit_end and returns the count. */
int64_t agpt_b200_plan_units(const agpt_plan *p, int level, int64_t cap, int64_t *unit_begin,
                             int64_t *unit_end);
/* Longest-processing-time assignment of units to ranks; rank_of_unit[u] in [0, n_ranks). */
int agpt_b200_partition_lpt(const int64_t *unit_weight, int64_t n_units, int n_ranks,
                            int32_t *rank_of_unit);

/* Launch groups of one rank: its units (depth-first [begin, end) ranges of a plan, e.g. from agpt_b200_plan_units; the
 * units with unit_rank[u] == rank, all of them if unit_rank is NULL) packed in order into forests of at most
 * group_rows rows -- the chunker of src/cuda/agpt_train.cu:4424-4443 on whole units.  A unit that does not start at
 * depth 1 is preceded by its ancestor chain as context rows (trained == 0: attended and differentiated through, but
 * they carry no loss), so every query finds its whole chain inside the group.  Per group: parent (local row index, -1
 * for roots; rows are in depth-first order, so it can go straight to agpt_b200_plan_create), row (the plan's
 * depth-first position of each row), trained, unit_of_row (index of the row's unit inside the group). */
typedef struct agpt_groups agpt_groups;
typedef struct {
    int64_t n;
    int32_t n_units;
    const int32_t *parent;
    const int64_t *row;
    const uint8_t *trained;
    const int32_t *unit_of_row;
} agpt_group_info;
int agpt_b200_groups_create(const agpt_plan *p, const int64_t *unit_begin, const int64_t *unit_end,
                            const int32_t *unit_rank, int64_t n_units, int rank, int64_t group_rows, agpt_groups **out);
int64_t agpt_b200_groups_count(const agpt_groups *g);
int agpt_b200_groups_get(const agpt_groups *g, int64_t i, agpt_group_info *out);
void agpt_b200_groups_free(agpt_groups *g);


/* ---- device kernels (all asynchronous on `stream`, a cudaStream_t passed as void*) ---- */

/* Row gather: dst[i, :] = src[index[i], :] (float32 rows of `cols`).  Used to bring
 * id-ordered activations into depth-first order and back. */
int agpt_b200_gather_rows(const float *d_src, const int32_t *d_index, float *d_dst, int64_t n, int cols,
                          void *stream);

/* Replaces build_rope_cache's host loop (src/cuda/agpt_train.cu:2298-2321): cos/sin [max_seq, head_dim],
 * theta = pos / base^(2i/head_dim) in float32 (powf, cosf, sinf), each value stored at 2i and 2i+1. */
int agpt_b200_rope_table(float *cos_out, float *sin_out, int max_seq, int head_dim, float base);

/* Replaces rope_batched_kernel / rope_batched_inverse_kernel (src/cuda/agpt_train.cu:1305-1351):
 * x [n, n_heads*head_dim] rotated in place, pair (2i, 2i+1) of each head by pos[row]. */
int agpt_b200_rope(float *d_x, const int32_t *d_pos, const float *d_cos, const float *d_sin, int64_t n,
                   int n_heads, int head_dim, int inverse, void *stream);
/* The same for two matrices of one shape that share the row positions (q and k, or their gradients), in one launch. */
int agpt_b200_rope_pair(float *d_a, float *d_b, const int32_t *d_pos, const float *d_cos, const float *d_sin, int64_t n,
                        int n_heads, int head_dim, int inverse, void *stream);

/* Replace cuda_layer_norm_forward / cuda_layer_norm_backward of the reference's kernel dependency (declared
 * src/cuda/agpt_train.cu:50-55; called :4671, :4762, :4801, :4850, :4907, :5066), with the arithmetic the reference
 * states on CPU (src/agpt/incremental_forward.cr:143-163, src/agpt/batched_depth_backward.cr:751-799): float32 mean
 * and biased variance, std_inv = 1/sqrt(var + 1e-5); output = norm*gamma + beta; norm_out and std_inv_out are the
 * saved state.  Backward: dx may alias grad; dgamma and dbeta are accumulated into, in a fixed order.  cols must
 * be a multiple of 4, at most 1024.  The legacy symbols run on the default stream and keep a per-device scratch. */
void cuda_layer_norm_forward(const float *input, float *output, float *norm_out, float *std_inv_out,
                             const float *gamma, const float *beta, int rows, int cols);
void cuda_layer_norm_backward(const float *grad, const float *norm, const float *std_inv, const float *gamma,
                              float *dx, float *dgamma, float *dbeta, int rows, int cols);
int agpt_b200_layer_norm_fwd(const float *d_x, float *d_y, float *d_norm, float *d_std_inv, const float *d_gamma,
                             const float *d_beta, int64_t rows, int cols, void *stream);
int agpt_b200_layer_norm_bwd(const float *d_grad, const float *d_norm, const float *d_std_inv, const float *d_gamma,
                             float *d_dx, float *d_dgamma, float *d_dbeta, int64_t rows, int cols, void *d_workspace,
                             int64_t workspace_bytes, void *stream);
/* The same with d_add[rows, cols] (NULL: none) added to dx: the gradient that reaches the normalised rows' input by
 * the residual path (the reference adds the two in its own pass, src/cuda/agpt_train.cu:4907-4909, :5066-5068).
 * d_add may be d_dx. */
int agpt_b200_layer_norm_bwd_add(const float *d_grad, const float *d_norm, const float *d_std_inv, const float *d_gamma,
                                 const float *d_add, float *d_dx, float *d_dgamma, float *d_dbeta, int64_t rows, int cols,
                                 void *d_workspace, int64_t workspace_bytes, void *stream);
int64_t agpt_b200_layer_norm_bwd_workspace_bytes(int64_t rows, int cols);

/* Replace the row-wise kernels of the reference's kernel dependency (declared src/cuda/agpt_train.cu:48-49,
 * :56-63; called :4646, :4677-4683, :4754, :4768-4772, :4805, :4893, :5073) and its bias_grad_accum_kernel
 * (:1774-1797).  Legacy symbols: void, default stream, 32-bit sizes, same argument order.
 *   cuda_bias_add              data += bias (row broadcast), in place
 *   cuda_fused_bias_relu       output = max(input + bias, 0); mask = 1.0 where output > 0 else 0.0 (output may alias input)
 *   cuda_relu_backward         output = grad where mask > 0 else 0 (so the saved activation works as the mask too)
 *   cuda_softmax_rows          row softmax;   cuda_softmax_backward   result = s * (ds - sum_c s*ds)
 *   cuda_embedding_gather      output[i] = token_emb[ids[i]] (ids < 0 give a zero row)
 *   cuda_embedding_scatter_add d_token_emb[ids[i]] += grad[i] with atomic adds (the vocabulary size is not an argument);
 *                              agpt_b200_embedding_grad is the repeatable form. */
void cuda_bias_add(float *data, const float *bias, int rows, int cols);
void cuda_fused_bias_relu(const float *input, const float *bias, float *output, float *mask, int rows, int cols);
void cuda_relu_backward(const float *grad, const float *mask, float *output, int n);
void cuda_softmax_rows(const float *input, float *output, int rows, int cols);
void cuda_softmax_backward(const float *s, const float *ds, float *result, int rows, int cols);
void cuda_embedding_gather(const float *token_emb, const int *ids, float *output, int seq_len, int d_model);
void cuda_embedding_scatter_add(const float *grad, const int *ids, float *d_token_emb, int seq_len, int d_model);
/* Native forms with a stream and 64-bit row counts.  bias_act: relu != 0 selects bias + ReLU, d_mask may be NULL.
 * col_sum: d_out[c] = (accumulate ? d_out[c] : 0) + scale * sum_r g[r][c], the bias gradient; with d_act != NULL the
 * gradient is first masked by d_act > 0 and the masked gradient written to d_grad_out (may alias d_grad): ReLU
 * backward and the bias gradient of the layer below it in one pass.  embedding_grad: the gradient of the embedding
 * table from per-block partial tables added in a fixed order (vocab up to 400).  Both reductions repeat bit for bit. */
int agpt_b200_bias_act(const float *d_in, const float *d_bias, float *d_out, float *d_mask, int64_t rows, int cols,
                       int relu, void *stream);
int agpt_b200_relu_bwd(const float *d_grad, const float *d_mask, float *d_out, int64_t n, void *stream);
int agpt_b200_col_sum(const float *d_grad, const float *d_act, float *d_grad_out, int64_t rows, int cols, float scale,
                      int accumulate, float *d_out, void *d_workspace, int64_t workspace_bytes, void *stream);
int64_t agpt_b200_col_sum_workspace_bytes(int64_t rows, int cols);
int agpt_b200_softmax_rows(const float *d_in, float *d_out, int64_t rows, int cols, void *stream);
int agpt_b200_softmax_bwd(const float *d_s, const float *d_ds, float *d_out, int64_t rows, int cols, void *stream);
int agpt_b200_embedding_gather(const float *d_emb, const int32_t *d_ids, float *d_out, int64_t n, int d_model,
                               int vocab, void *stream);
int agpt_b200_embedding_grad(const float *d_grad, const int32_t *d_ids, float *d_emb_grad, int64_t n, int d_model,
                             int vocab, int accumulate, void *d_workspace, int64_t workspace_bytes, void *stream);
int64_t agpt_b200_embedding_grad_workspace_bytes(int64_t n, int d_model, int vocab);

/* Replace the optimizer kernels of the reference's kernel dependency (declared src/cuda/agpt_train.cu:64-72;
 * called in the order clip, update, decay at :5135-5162 and :5190-5214).  The dependency's source is not part of
 * the reference; the rules implemented are
 *   sgd p -= lr*g;   momentum m = beta*m + g, p -= lr*m;   rmsprop s = beta*s + (1-beta)*g*g, p -= lr*g/(sqrt(s)+eps);
 *   adam m = b1*m + (1-b1)*g, v = b2*v + (1-b2)*g*g, p -= lr*(m/(1-b1^t))/(sqrt(v/(1-b2^t))+eps), t from 1;
 *   weight decay p -= lr*wd*p;   clip g *= max_norm/||g|| when ||g|| > max_norm (norm_scratch[0] receives ||g||;
 *   partials_scratch holds ceil(n/256) floats as the reference allocates, at most 1024 are used). */
void cuda_adam_bulk(float *params, float *grads, float *m, float *v, float lr, float beta1, float beta2, float eps,
                    int t, int n);
void cuda_sgd_bulk(float *params, float *grads, float lr, int n);
void cuda_momentum_bulk(float *params, float *grads, float *m, float lr, float beta, int n);
void cuda_rmsprop_bulk(float *params, float *grads, float *s, float lr, float beta, float eps, int n);
void cuda_weight_decay(float *params, float lr, float wd, int n);
void cuda_grad_clip_by_norm(float *grads, float max_norm, int n, float *partials_scratch, float *norm_scratch);
/* The whole step in two launches over the flat buffers: clip (clip_norm > 0; needs d_scratch of
 * agpt_b200_optimizer_scratch_bytes(), whose last float receives the gradient norm), update by `kind`, decay
 * (weight_decay > 0), and clearing of the gradients (zero_grads != 0).  beta1 is the momentum / first-moment
 * coefficient, beta2 the RMSProp / second-moment coefficient. */
#define AGPT_OPT_SGD 0
#define AGPT_OPT_MOMENTUM 1
#define AGPT_OPT_RMSPROP 2
#define AGPT_OPT_ADAM 3
int agpt_b200_optimizer_step(int kind, float *d_params, float *d_grads, float *d_m, float *d_v, int64_t n, float lr,
                             float beta1, float beta2, float eps, int t, float weight_decay, float clip_norm,
                             int zero_grads, void *d_scratch, void *stream);
int64_t agpt_b200_optimizer_scratch_bytes(void);

/* Replaces the cublasSgemm calls of the dense projections (src/cuda/agpt_train.cu:4675-4683, :4752, :4766-4771,
 * :4803, :4840-5061) with a tensor-core GEMM of float32-level accuracy (three TF32 MMAs per product).  Row-major:
 *     out[M, N] = act(alpha * op(A)[M, K] * op(B)[K, N] + beta * C + bias)
 * trans_a / trans_b select A^T / B^T (not both).  d_c (with beta != 0) is a source matrix such as the residual
 * stream, or the running sum of the input gradients of several projections of the same rows (:5026-5061); it may be
 * d_out itself.  d_bias is a row added to every row, relu != 0 applies max(., 0); each may be absent (NULL / 0).  split_k > 1
 * cuts K into slices (for weight gradients, whose K is the number of trie positions; no bias or activation then): the
 * slices run as one batched GEMM into partial matrices in d_workspace (agpt_b200_gemm_f32_workspace_bytes, 0 when
 * split_k == 1) and are added in slice order, so the result is repeatable bit for bit.  Pointers and leading
 * dimensions must be multiples of 4 floats. */
int agpt_b200_gemm_f32(int trans_a, int trans_b, int M, int N, int K, float alpha, const float *d_a, int lda,
                       const float *d_b, int ldb, float beta, const float *d_c, int ldc, const float *d_bias, int relu,
                       float *d_out, int ldd, int split_k, void *d_workspace, int64_t workspace_bytes, void *stream);
int64_t agpt_b200_gemm_f32_workspace_bytes(int trans_a, int trans_b, int M, int N, int K, int split_k);
/* Two implementations compute agpt_b200_gemm_f32: 1 (default) tcgen05 MMAs on bfloat16 splits of the operands with
 * TMA loads and tensor-memory accumulators; 0 mma.sync with three TF32 products (also set by the environment
 * variable AGPT_B200_GEMM_IMPL=0).  Both agree with a float32 GEMM to about 1e-6. */
int agpt_b200_set_gemm_impl(int impl);

/* Replaces kv_scatter_kernel_bf16 (src/cuda/agpt_train.cu:1537-1554) for a store laid out in
 * depth-first order: d_store[i, :] = bf16(d_src[i, :]). */
int agpt_b200_kv_store_write_bf16(const float *d_src, void *d_store_bf16, int64_t n, int cols, void *stream);

/* Replaces kv_gather + cuda_batched_varlen_attention(_L_queries) (src/cuda/agpt_train.cu:4689-4749,
 * src/agpt/batched_depth_forward.cr:836-971).  d_q, d_out [n, H*hd] float32 in depth-first order;
 * d_k, d_v the KV store [n, H*hd] of kv_dtype; d_lse [n, H] = log sum exp of the scaled scores. */
int agpt_b200_attn_fwd(const agpt_plan *p, const float *d_q, const void *d_k, const void *d_v, int kv_dtype,
                       float *d_out, float *d_lse, int n_heads, int head_dim, float scale, void *stream);

/* Replaces cuda_batched_varlen_attention(_L_queries)_backward + kv_scatter_add
 * (src/cuda/agpt_train.cu:4982-5035, :1896-1935; src/agpt/batched_depth_backward.cr:605-695).
 * d_dq, d_dk, d_dv [n, H*hd] float32 fully written; d_dk/d_dv hold, per node, the sum over the node
 * itself and all its descendants, accumulated in a fixed order.  d_workspace: scratch of
 * agpt_b200_attn_bwd_workspace_bytes(). */
int agpt_b200_attn_bwd(const agpt_plan *p, const float *d_q, const void *d_k, const void *d_v, int kv_dtype,
                       const float *d_out, const float *d_lse, const float *d_dout, float *d_dq, float *d_dk,
                       float *d_dv, void *d_workspace, int64_t workspace_bytes, int n_heads, int head_dim,
                       float scale, void *stream);

/* agpt_b200_attn_bwd with a choice of which attention pairs feed dK/dV; dQ always takes every attended key.  The
 * reference has three behaviours and this entry point reproduces each:
 *   AGPT_GRAD_FULL         a node's dK/dV sum over the node itself and all its descendants (persistent
 *                          accumulators: src/agpt/incremental_backward.cr:101-147 + src/agpt/node_state.cr:58-74);
 *   AGPT_GRAD_LOCAL_DEPTH  only the node's own query (the accumulators are dropped after each depth and subtrie:
 *                          src/agpt/trie_walk_trainer.cr:189);
 *   AGPT_GRAD_OWN_EDGE     the queries on the key's own radix edge (the ancestor part of the packed dK/dV is dropped:
 *                          src/cuda/agpt_train.cu:5016-5020).  d_edge_first [n] int32: for every position, the
 *                          depth-first position of the first char of its radix edge (ignored by the other modes). */
#define AGPT_GRAD_FULL 0
#define AGPT_GRAD_LOCAL_DEPTH 1
#define AGPT_GRAD_OWN_EDGE 2
int agpt_b200_attn_bwd_mode(const agpt_plan *p, const float *d_q, const void *d_k, const void *d_v, int kv_dtype,
                            const float *d_out, const float *d_lse, const float *d_dout, float *d_dq, float *d_dk,
                            float *d_dv, void *d_workspace, int64_t workspace_bytes, int n_heads, int head_dim,
                            float scale, int grad_mode, const int32_t *d_edge_first, void *stream);

/* Selects the kernel family behind agpt_b200_attn_fwd/_bwd: 1 = tensor cores (mma.sync TF32 with error
 * compensation, tiles of 64; the default), 0 = FP32 FMA.  Both meet the same parity tolerances; the switch
 * exists for A/B measurement.  Also read once from the environment variable AGPT_B200_ATTN_IMPL. */
int agpt_b200_set_attn_impl(int impl);

/* Selects between the two tensor-core kernel pairs for a float32 KV store and head_dim 32 or 64.  whole_tile 1
 * (default): forward and backward keep the tile's Q (and dO) rows and all its key rows in shared memory, converted
 * once to split half precision (x * 2^e = hi + lo, fp16 each, e per tile, head and tensor; three m16n8k16 products
 * give the accuracy of three TF32 products), every fragment one ldmatrix, and the backward's warps run independent
 * row and key items with no barrier in their loops.  Used whenever four (head_dim 32) or two (head_dim 64) blocks
 * of the backward fit one SM, i.e. up to about 150 / 128 keys per tile (depth <= ~90 / 65); deeper plans and head_dim 16
 * take the chunked TF32 kernels, and so does the head_dim-64 forward (the chunked one measured faster there).  With a
 * bf16 store the whole-tile backward runs at head_dim 32 (single fp16 products: the store's own rounding is coarser;
 * AGPT_B200_ATTN_TILE_BF16=0 in the environment keeps the chunked kernel), everything else chunked.  whole_tile 0:
 * always the chunked kernels.  bwd_warps = 4 (default), 6 or 8 warps per block of the whole-tile backward, 3 = four
 * warps with three blocks per SM.  Same results within the parity tolerance either way; the switch exists for A/B
 * measurement.  Also read once from AGPT_B200_ATTN_TILE and AGPT_B200_BWD_WARPS; AGPT_B200_FWD_BLOCKS=5 runs the
 * head_dim-32 forward with five blocks per SM instead of six. */
int agpt_b200_set_attn_variant(int whole_tile, int bwd_warps);

/* No counterpart in the reference.  agpt_b200_attn_bwd for callers that cannot allocate device memory
 * when the backward runs -- a runtime that claimed the whole GPU at start-up and sub-allocates from its own
 * pool, or a step whose set of buffers is frozen -- and therefore have no workspace to pass.  The partial
 * dK/dV rows go to an array built into the library instead: agpt_b200_static_scratch_bytes() bytes
 * (64 MiB), resident on every GPU that loads the library for as long as the process lives.  Same inputs,
 * outputs and results as agpt_b200_attn_bwd.  A plan whose agpt_b200_attn_bwd_workspace_bytes() exceeds the
 * array is refused with AGPT_E_LIMIT.  The call performs no cudaMalloc/cudaFree and calls no allocating
 * routine.  The plan's device must be the current device.  The first call on each device looks up the
 * array's device address (cudaGetSymbolAddress), so make that first call outside any stream capture.  All
 * calls on one GPU share the array: two calls whose kernels may overlap (different streams, or different
 * host threads) race on it -- keep them on one stream or serialise them.  Nothing in the array has to be
 * cleared between calls: every element a call reads it has written first. */
int agpt_b200_attn_bwd_static(const agpt_plan *p, const float *d_q, const void *d_k, const void *d_v,
                              int kv_dtype, const float *d_out, const float *d_lse, const float *d_dout,
                              float *d_dq, float *d_dk, float *d_dv, int n_heads, int head_dim, float scale,
                              void *stream);
int64_t agpt_b200_static_scratch_bytes(void);

/* Device status word of the current GPU (waits for the work issued so far): 0 when every kernel ran to completion.
 * Bit 0: a bounded wait for a bulk asynchronous copy in the loss kernel ran out; the affected rows were not
 * written.  Kernels never trap; this word is how a failure on the device reaches the host. */
int agpt_b200_device_status(int32_t *status_out);

/* Replaces agpt_loss_per_query_kernel (src/cuda/agpt_train.cu:2069-2216).  Same arguments. */
int agpt_b200_loss_per_query(const float *d_logits, const int32_t *d_query_to_node,
                             const int32_t *d_query_offsets, const int32_t *d_radix_ids,
                             const int32_t *d_token_ids, const int32_t *d_counts_offset,
                             const int32_t *d_counts_tok, const int32_t *d_counts_val,
                             const float *d_mass_weights, float *d_dlogits, float *d_loss, int64_t T_q, int V,
                             float entropy_lambda, float intermediate_weight, int ce_only, void *stream);

/* Replaces agpt_loss_kernel (src/cuda/agpt_train.cu:1947-2044). */
int agpt_b200_loss_per_node(const float *d_logits, const int32_t *d_node_ids, const int32_t *d_counts_offset,
                            const int32_t *d_counts_tok, const int32_t *d_counts_val, float *d_dlogits,
                            float *d_loss, int64_t N, int V, void *stream);

/* Host-buffer convenience of the same step (what gpu_batched_attention /
 * gpu_attention_backward_depth do around the kernels, src/agpt/batched_depth_forward.cr:745-823,
 * src/agpt/batched_depth_backward.cr:453-500): uploads q, k, v, d_out from host memory, runs forward
 * and backward, downloads out, lse, dq, dk, dv.  Upload, compute and download run as a pipeline over row chunks
 * on three internal streams; the call returns when everything is on the host.  The overlap needs page-locked host
 * buffers (cudaHostAlloc / cudaHostRegister): with pageable memory every copy is staged by the driver and blocks the
 * host thread, so the three stages run one after the other (results are the same).  If a step fails midway the
 * call waits for the copies already queued before it returns the error, so the host buffers are never touched
 * after the call has returned.  The device arena is allocated at the first call on a plan and kept until
 * agpt_b200_plan_destroy, so one plan must not be used by two host threads at once. */
int agpt_b200_attn_fwd_bwd_host(const agpt_plan *p, const float *h_q, const float *h_k, const float *h_v,
                                const float *h_dout, float *h_out, float *h_lse, float *h_dq, float *h_dk,
                                float *h_dv, int kv_dtype, int n_heads, int head_dim, float scale);

#ifdef __cplusplus
}
#endif
#endif /* AGPT_B200_H */
