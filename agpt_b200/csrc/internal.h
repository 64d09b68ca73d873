// Shared between the host walker code and the CUDA translation unit of libagpt_b200.
#pragma once
#include <cstdint>
#include <vector>

#define AGPT_REDUCE_SEG 128   // tiles summed by one warp of the dK/dV reduction before a second pass

int agpt_set_error(int code, const char *fmt, ...);

// Radix trie with the reference's node numbering (ids in the builder's breadth-first emission order), counts, edge
// mass and char positions.
struct agpt_trie {
    int32_t radix_count = 0, n_depth_files = 0;
    int64_t total_edge_chars = 0, leveled_nodes = 0;
    std::vector<int32_t> parent, first_char_depth, edge_len, edge_mass, endpoint_depth, subtree_key, edge_start;
    std::vector<int64_t> edge_off, cnt_off;
    std::vector<int32_t> edge_tok, cnt_tok, cnt_val;
    void finish_char_positions() {
        // char positions follow depth-file order (src/cuda/agpt_train.cu:813-846)
        edge_start.assign(radix_count, 0);
        std::vector<int64_t> per_depth(n_depth_files + 1, 0);
        for (int32_t r = 1; r < radix_count; r++) per_depth[endpoint_depth[r] + 1] += edge_len[r];
        for (int d = 0; d < n_depth_files; d++) per_depth[d + 1] += per_depth[d];
        for (int32_t r = 1; r < radix_count; r++) {
            edge_start[r] = (int32_t)per_depth[endpoint_depth[r]];
            per_depth[endpoint_depth[r]] += edge_len[r];
        }
    }
};

// Walker plan: a tree laid out in depth-first pre-order.  Position i's subtree is the
// interval [i, sub_end[i]); a is an ancestor-or-self of i iff a <= i < sub_end[a].  Queries
// are processed in tiles of tile_m consecutive positions; a tile's keys are the ancestor
// chain of its first position (chain_ids, root side first, chain_off per tile) plus the
// tile's own rows.
struct agpt_plan {
    int64_t n = 0;
    int32_t tile_m = 64;
    int64_t n_tiles = 0;
    int32_t max_depth = 0;
    int64_t sum_depth = 0, sum_group_prefix = 0, n_groups = 0, n_reduce_nodes = 0, n_multi_items = 0;
    std::vector<int32_t> dfs_to_node, node_to_dfs, parent_dfs, depth, sub_end;
    std::vector<int64_t> chain_off;
    std::vector<int32_t> chain_ids, chain_end;   // chain_end[j] = sub_end[chain_ids[j]]
    // dK/dV reduction work list: item = (node, inclusive tile range); slot >= 0 when the node's range
    // is cut into several items whose sums meet in a second pass
    std::vector<int32_t> item_node, item_t0, item_t1, item_slot;
    std::vector<int32_t> multi_node, multi_count;
    std::vector<int64_t> multi_first;          // first segment slot of each multi-segment node (its slots are consecutive)
    // device copies (owned)
    int device = -1;
    int32_t *d_depth = nullptr, *d_sub_end = nullptr, *d_chain_ids = nullptr, *d_chain_end = nullptr;
    int64_t *d_chain_off = nullptr, *d_multi_first = nullptr;
    int32_t *d_item_node = nullptr, *d_item_t0 = nullptr, *d_item_t1 = nullptr, *d_item_slot = nullptr;
    int32_t *d_multi_node = nullptr, *d_multi_count = nullptr;
    // host-buffer step (agpt_b200_attn_fwd_bwd_host): device arena, three streams (upload, compute, download) and
    // per-chunk events; created at first use, kept for later calls, released with the plan
    void *host_arena = nullptr;
    size_t host_arena_bytes = 0;
    void *host_streams[3] = {nullptr, nullptr, nullptr};
    std::vector<void *> host_events;
    void *host_fix = nullptr;                  // pinned staging for rows re-downloaded at the end of a host-buffer step
    size_t host_fix_bytes = 0;
    ~agpt_plan();
};

int agpt_plan_upload(agpt_plan *p, int device);

// tcgen05 float32 GEMM (gemm_sm100.cu): D[l] = act(alpha * op(A[l]) * op(B[l]) + beta * C + bias row), l < L batches
bool agpt_gemm_sm100_takes(int trans_a, int trans_b, int relu, int has_source);
int agpt_gemm_sm100(int trans_a, int trans_b, int M, int N, int K, int L, float alpha, const float *A, int64_t lda, int64_t batch_a,
                    const float *B, int64_t ldb, int64_t batch_b, const float *bias, int relu, float beta, const float *C, int64_t ldc,
                    float *D, int64_t ldd, int64_t batch_d, void *stream);
