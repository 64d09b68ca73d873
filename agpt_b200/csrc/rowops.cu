// The small row-wise kernels of the dense step around the trie attention: bias add, bias + ReLU, ReLU backward,
// bias gradient (column sums), row softmax and its backward, embedding gather and its gradient.  They replace the
// kernel dependency the reference declares at src/cuda/agpt_train.cu:47-63 (cuda_softmax_rows, cuda_softmax_backward,
// cuda_bias_add, cuda_fused_bias_relu, cuda_relu_backward, cuda_embedding_gather, cuda_embedding_scatter_add) and
// its bias_grad_accum_kernel (:1774-1797).  All of them are bound by HBM traffic: every kernel touches each element
// once with 16-byte accesses where the row width allows, grids are sized from the SM count, and the reductions
// (column sums, embedding gradient) run as per-block partials added in a fixed order, so results repeat bit for bit.
#include <cuda_runtime.h>

#include <cstdint>

#include "../../include/agpt_b200.h"
#include "internal.h"

namespace {

int sm_count() {
    static int cached[64] = {0};
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev < 0 || dev >= 64) return 148;
    if (!cached[dev]) cudaDeviceGetAttribute(&cached[dev], cudaDevAttrMultiProcessorCount, dev);
    return cached[dev] > 0 ? cached[dev] : 148;
}

int launch_status(const char *who) {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return agpt_set_error(AGPT_E_CUDA, "%s: %s", who, cudaGetErrorString(e));
    return AGPT_OK;
}

unsigned grid_for(int64_t work_items, int per_block, int blocks_per_sm) {
    int64_t want = (work_items + per_block - 1) / per_block;
    int64_t cap = (int64_t)sm_count() * blocks_per_sm;
    return (unsigned)(want < 1 ? 1 : (want < cap ? want : cap));
}

// ---- bias add / bias + ReLU / ReLU backward ------------------------------------------------------------------
// MODE 0: out = in + bias; MODE 1: out = max(in + bias, 0), mask = (out > 0)
template <int MODE, bool VEC>
__global__ void __launch_bounds__(256) bias_kernel(const float *__restrict__ in, const float *__restrict__ bias, float *__restrict__ out,
                                                    float *__restrict__ mask, int64_t rows, int cols) {
    if (VEC) {
        const int c4 = cols >> 2;
        const int64_t n4 = rows * c4;
        for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (int64_t)gridDim.x * blockDim.x) {
            int c = (int)(i % c4);
            float4 v = reinterpret_cast<const float4 *>(in)[i];
            float4 b = __ldg(reinterpret_cast<const float4 *>(bias) + c);
            v.x += b.x; v.y += b.y; v.z += b.z; v.w += b.w;
            if (MODE == 1) {
                float4 m = make_float4(v.x > 0.f ? 1.f : 0.f, v.y > 0.f ? 1.f : 0.f, v.z > 0.f ? 1.f : 0.f, v.w > 0.f ? 1.f : 0.f);
                v.x = fmaxf(v.x, 0.f); v.y = fmaxf(v.y, 0.f); v.z = fmaxf(v.z, 0.f); v.w = fmaxf(v.w, 0.f);
                if (mask) reinterpret_cast<float4 *>(mask)[i] = m;
            }
            reinterpret_cast<float4 *>(out)[i] = v;
        }
    } else {
        const int64_t n = rows * cols;
        for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
            float v = in[i] + __ldg(bias + (int)(i % cols));
            if (MODE == 1) {
                if (mask) mask[i] = v > 0.f ? 1.f : 0.f;
                v = fmaxf(v, 0.f);
            }
            out[i] = v;
        }
    }
}

template <bool VEC>
__global__ void __launch_bounds__(256) relu_bwd_kernel(const float *__restrict__ grad, const float *__restrict__ mask,
                                                        float *__restrict__ out, int64_t n) {
    if (VEC) {
        const int64_t n4 = n >> 2;
        for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n4; i += (int64_t)gridDim.x * blockDim.x) {
            float4 g = reinterpret_cast<const float4 *>(grad)[i], m = reinterpret_cast<const float4 *>(mask)[i];
            // any positive mask entry passes the gradient: a 0/1 mask and the saved activation both work
            g.x = m.x > 0.f ? g.x : 0.f; g.y = m.y > 0.f ? g.y : 0.f; g.z = m.z > 0.f ? g.z : 0.f; g.w = m.w > 0.f ? g.w : 0.f;
            reinterpret_cast<float4 *>(out)[i] = g;
        }
    } else {
        for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x)
            out[i] = mask[i] > 0.f ? grad[i] : 0.f;
    }
}

bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }

// ---- column sums (bias gradient), optionally of a ReLU-masked gradient that is written back --------------------
// Block b owns rows [b*chunk, (b+1)*chunk); thread t owns column quad t % q and every (256/q)-th row of the chunk.
// partial[b][cols] is the block's sum; the finish kernel adds the blocks in order.
template <bool MASKED>
__global__ void __launch_bounds__(256) col_sum_kernel(const float *__restrict__ grad, const float *__restrict__ act, float *__restrict__ gout,
                                                       int64_t rows, int cols, int64_t chunk, float *__restrict__ partial) {
    extern __shared__ float4 s_part[];               // [256 / q][q]
    const int q = cols >> 2, lanes = 256 / q;
    const int c = threadIdx.x % q, lane = threadIdx.x / q;
    const int64_t r0 = (int64_t)blockIdx.x * chunk, r1 = (r0 + chunk < rows) ? r0 + chunk : rows;
    float4 acc = make_float4(0.f, 0.f, 0.f, 0.f);
    if (lane < lanes) {
        for (int64_t r = r0 + lane; r < r1; r += lanes) {
            float4 g = reinterpret_cast<const float4 *>(grad + r * cols)[c];
            if (MASKED) {
                float4 a = reinterpret_cast<const float4 *>(act + r * cols)[c];
                g.x = a.x > 0.f ? g.x : 0.f; g.y = a.y > 0.f ? g.y : 0.f; g.z = a.z > 0.f ? g.z : 0.f; g.w = a.w > 0.f ? g.w : 0.f;
                reinterpret_cast<float4 *>(gout + r * cols)[c] = g;
            }
            acc.x += g.x; acc.y += g.y; acc.z += g.z; acc.w += g.w;
        }
        s_part[lane * q + c] = acc;
    }
    __syncthreads();
    if (threadIdx.x < q) {
        float4 t = s_part[threadIdx.x];
        for (int l = 1; l < lanes; l++) {
            float4 p = s_part[l * q + threadIdx.x];
            t.x += p.x; t.y += p.y; t.z += p.z; t.w += p.w;
        }
        reinterpret_cast<float4 *>(partial + (int64_t)blockIdx.x * cols)[threadIdx.x] = t;
    }
}

// out[c] = (accumulate ? out[c] : 0) + scale * sum_b partial[b][c]
__global__ void __launch_bounds__(256) col_sum_finish_kernel(const float *__restrict__ partial, int blocks, int cols, float scale,
                                                              int accumulate, float *__restrict__ out) {
    int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= cols) return;
    float t = 0.f;
    for (int b = 0; b < blocks; b++) t += partial[(int64_t)b * cols + c];
    out[c] = (accumulate ? out[c] : 0.f) + scale * t;
}

// scalar fallback for widths that are not a multiple of 4 or exceed 1024: one block per column, as the reference
__global__ void __launch_bounds__(256) col_sum_scalar_kernel(const float *__restrict__ grad, int64_t rows, int cols, float scale,
                                                              int accumulate, float *__restrict__ out) {
    __shared__ float s[256];
    int c = blockIdx.x;
    float t = 0.f;
    for (int64_t r = threadIdx.x; r < rows; r += 256) t += grad[r * cols + c];
    s[threadIdx.x] = t;
    __syncthreads();
    for (int k = 128; k > 0; k >>= 1) {
        if (threadIdx.x < k) s[threadIdx.x] += s[threadIdx.x + k];
        __syncthreads();
    }
    if (threadIdx.x == 0) out[c] = (accumulate ? out[c] : 0.f) + scale * s[0];
}

int col_sum_blocks(int64_t rows) {
    int64_t b = (rows + 511) / 512;
    int64_t cap = (int64_t)sm_count() * 4;
    return (int)(b < 1 ? 1 : (b < cap ? b : cap));
}

// ---- row softmax and its backward: one warp per row ----------------------------------------------------------
__global__ void __launch_bounds__(256) softmax_rows_kernel(const float *__restrict__ in, float *__restrict__ out, int64_t rows, int cols) {
    const int lane = threadIdx.x & 31;
    for (int64_t r = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5); r < rows; r += (int64_t)gridDim.x * 8) {
        const float *x = in + r * cols;
        float mx = -INFINITY;
        for (int c = lane; c < cols; c += 32) mx = fmaxf(mx, x[c]);
        for (int o = 16; o; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        float sum = 0.f;
        for (int c = lane; c < cols; c += 32) sum += expf(x[c] - mx);
        for (int o = 16; o; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
        const float inv = 1.f / sum;
        for (int c = lane; c < cols; c += 32) out[r * cols + c] = expf(x[c] - mx) * inv;
    }
}

// result = s * (ds - sum_c s*ds)
__global__ void __launch_bounds__(256) softmax_bwd_kernel(const float *__restrict__ s, const float *__restrict__ ds, float *__restrict__ res,
                                                           int64_t rows, int cols) {
    const int lane = threadIdx.x & 31;
    for (int64_t r = (int64_t)blockIdx.x * 8 + (threadIdx.x >> 5); r < rows; r += (int64_t)gridDim.x * 8) {
        const float *sr = s + r * cols, *dr = ds + r * cols;
        float dot = 0.f;
        for (int c = lane; c < cols; c += 32) dot += sr[c] * dr[c];
        for (int o = 16; o; o >>= 1) dot += __shfl_xor_sync(0xffffffffu, dot, o);
        for (int c = lane; c < cols; c += 32) res[r * cols + c] = sr[c] * (dr[c] - dot);
    }
}

// ---- embedding gather and gradient ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256) embedding_gather_kernel(const float *__restrict__ emb, const int *__restrict__ ids,
                                                                float *__restrict__ out, int64_t n, int d, int vocab) {
    const int64_t total = n * d;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        int64_t r = i / d;
        int id = ids[r];
        out[i] = (id >= 0 && (vocab <= 0 || id < vocab)) ? emb[(int64_t)id * d + (i - r * d)] : 0.f;
    }
}

// legacy form (vocabulary size unknown): atomic adds into the table
__global__ void __launch_bounds__(256) embedding_scatter_atomic_kernel(const float *__restrict__ grad, const int *__restrict__ ids,
                                                                        float *__restrict__ demb, int64_t n, int d) {
    const int64_t total = n * d;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        int64_t r = i / d;
        int id = ids[r];
        if (id >= 0) atomicAdd(demb + (int64_t)id * d + (i - r * d), grad[i]);
    }
}

// Native form: block b sums its rows [b*chunk, ...) into a [vocab][DT] table in shared memory for the column tile
// blockIdx.y (thread = column, rows visited in order: no atomics), and writes it to partial[b]; the finish kernel
// adds the blocks in order.
__global__ void __launch_bounds__(128) embedding_grad_kernel(const float *__restrict__ grad, const int *__restrict__ ids, int64_t n, int d,
                                                              int vocab, int64_t chunk, float *__restrict__ partial) {
    extern __shared__ float s_tab[];                  // [vocab][128]
    const int c = blockIdx.y * 128 + threadIdx.x;
    for (int v = 0; v < vocab; v++) s_tab[v * 128 + threadIdx.x] = 0.f;
    const int64_t r0 = (int64_t)blockIdx.x * chunk, r1 = (r0 + chunk < n) ? r0 + chunk : n;
    if (c < d) {
        for (int64_t r = r0; r < r1; r++) {
            int id = __ldg(ids + r);
            if (id >= 0 && id < vocab) s_tab[id * 128 + threadIdx.x] += grad[r * d + c];
        }
        float *dst = partial + (int64_t)blockIdx.x * vocab * d;
        for (int v = 0; v < vocab; v++) dst[(int64_t)v * d + c] = s_tab[v * 128 + threadIdx.x];
    }
}

__global__ void __launch_bounds__(256) embedding_grad_finish_kernel(const float *__restrict__ partial, int blocks, int64_t vd, int accumulate,
                                                                     float *__restrict__ demb) {
    int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= vd) return;
    float t = 0.f;
    for (int b = 0; b < blocks; b++) t += partial[(int64_t)b * vd + i];
    demb[i] = (accumulate ? demb[i] : 0.f) + t;
}

int embedding_blocks(int64_t n) {
    int64_t b = (n + 2047) / 2048;
    int64_t cap = (int64_t)sm_count() * 2;
    return (int)(b < 1 ? 1 : (b < cap ? b : cap));
}

}  // namespace

// ---- native entry points ---------------------------------------------------------------------------------------

extern "C" int agpt_b200_bias_act(const float *d_in, const float *d_bias, float *d_out, float *d_mask, int64_t rows, int cols, int relu,
                                  void *stream) {
    if (!d_in || !d_bias || !d_out || rows < 0 || cols <= 0) return agpt_set_error(AGPT_E_ARG, "bias_act: bad argument");
    if (rows == 0) return AGPT_OK;
    cudaStream_t st = (cudaStream_t)stream;
    const bool vec = cols % 4 == 0 && aligned16(d_in) && aligned16(d_out) && aligned16(d_bias) && (!d_mask || aligned16(d_mask));
    unsigned g = grid_for(rows * cols / (vec ? 4 : 1), 256, 16);
    if (relu) {
        if (vec) bias_kernel<1, true><<<g, 256, 0, st>>>(d_in, d_bias, d_out, d_mask, rows, cols);
        else bias_kernel<1, false><<<g, 256, 0, st>>>(d_in, d_bias, d_out, d_mask, rows, cols);
    } else {
        if (vec) bias_kernel<0, true><<<g, 256, 0, st>>>(d_in, d_bias, d_out, nullptr, rows, cols);
        else bias_kernel<0, false><<<g, 256, 0, st>>>(d_in, d_bias, d_out, nullptr, rows, cols);
    }
    return launch_status("bias_act");
}

extern "C" int agpt_b200_relu_bwd(const float *d_grad, const float *d_mask, float *d_out, int64_t n, void *stream) {
    if (!d_grad || !d_mask || !d_out || n < 0) return agpt_set_error(AGPT_E_ARG, "relu_bwd: bad argument");
    if (n == 0) return AGPT_OK;
    cudaStream_t st = (cudaStream_t)stream;
    const bool vec = n % 4 == 0 && aligned16(d_grad) && aligned16(d_mask) && aligned16(d_out);
    unsigned g = grid_for(n / (vec ? 4 : 1), 256, 16);
    if (vec) relu_bwd_kernel<true><<<g, 256, 0, st>>>(d_grad, d_mask, d_out, n);
    else relu_bwd_kernel<false><<<g, 256, 0, st>>>(d_grad, d_mask, d_out, n);
    return launch_status("relu_bwd");
}

extern "C" int64_t agpt_b200_col_sum_workspace_bytes(int64_t rows, int cols) {
    if (rows < 0 || cols <= 0) return agpt_set_error(AGPT_E_ARG, "col_sum_workspace_bytes: bad argument");
    return (int64_t)col_sum_blocks(rows) * cols * 4;
}

extern "C" int agpt_b200_col_sum(const float *d_grad, const float *d_act, float *d_grad_out, int64_t rows, int cols, float scale,
                                 int accumulate, float *d_out, void *d_workspace, int64_t workspace_bytes, void *stream) {
    if (!d_grad || !d_out || rows < 0 || cols <= 0 || (d_act && !d_grad_out)) return agpt_set_error(AGPT_E_ARG, "col_sum: bad argument");
    cudaStream_t st = (cudaStream_t)stream;
    const bool vec = cols % 4 == 0 && cols <= 1024 && aligned16(d_grad) && (!d_act || (aligned16(d_act) && aligned16(d_grad_out)));
    if (!vec) {
        if (d_act) {
            int rc = agpt_b200_relu_bwd(d_grad, d_act, d_grad_out, rows * cols, stream);
            if (rc) return rc;
            d_grad = d_grad_out;
        }
        col_sum_scalar_kernel<<<cols, 256, 0, st>>>(d_grad, rows, cols, scale, accumulate, d_out);
        return launch_status("col_sum");
    }
    const int blocks = col_sum_blocks(rows);
    if (!d_workspace || workspace_bytes < (int64_t)blocks * cols * 4 || !aligned16(d_workspace))
        return agpt_set_error(AGPT_E_ARG, "col_sum: workspace too small (agpt_b200_col_sum_workspace_bytes)");
    const int64_t chunk = (rows + blocks - 1) / blocks;
    float *partial = (float *)d_workspace;
    const size_t smem = 256 * sizeof(float4);
    if (d_act) col_sum_kernel<true><<<blocks, 256, smem, st>>>(d_grad, d_act, d_grad_out, rows, cols, chunk, partial);
    else col_sum_kernel<false><<<blocks, 256, smem, st>>>(d_grad, nullptr, nullptr, rows, cols, chunk, partial);
    col_sum_finish_kernel<<<(cols + 255) / 256, 256, 0, st>>>(partial, blocks, cols, scale, accumulate, d_out);
    return launch_status("col_sum");
}

extern "C" int agpt_b200_softmax_rows(const float *d_in, float *d_out, int64_t rows, int cols, void *stream) {
    if (!d_in || !d_out || rows < 0 || cols <= 0) return agpt_set_error(AGPT_E_ARG, "softmax_rows: bad argument");
    if (rows == 0) return AGPT_OK;
    softmax_rows_kernel<<<grid_for(rows, 8, 8), 256, 0, (cudaStream_t)stream>>>(d_in, d_out, rows, cols);
    return launch_status("softmax_rows");
}

extern "C" int agpt_b200_softmax_bwd(const float *d_s, const float *d_ds, float *d_out, int64_t rows, int cols, void *stream) {
    if (!d_s || !d_ds || !d_out || rows < 0 || cols <= 0) return agpt_set_error(AGPT_E_ARG, "softmax_bwd: bad argument");
    if (rows == 0) return AGPT_OK;
    softmax_bwd_kernel<<<grid_for(rows, 8, 8), 256, 0, (cudaStream_t)stream>>>(d_s, d_ds, d_out, rows, cols);
    return launch_status("softmax_bwd");
}

extern "C" int agpt_b200_embedding_gather(const float *d_emb, const int32_t *d_ids, float *d_out, int64_t n, int d_model, int vocab,
                                          void *stream) {
    if (!d_emb || !d_ids || !d_out || n < 0 || d_model <= 0) return agpt_set_error(AGPT_E_ARG, "embedding_gather: bad argument");
    if (n == 0) return AGPT_OK;
    embedding_gather_kernel<<<grid_for(n * d_model, 256, 16), 256, 0, (cudaStream_t)stream>>>(d_emb, d_ids, d_out, n, d_model, vocab);
    return launch_status("embedding_gather");
}

extern "C" int64_t agpt_b200_embedding_grad_workspace_bytes(int64_t n, int d_model, int vocab) {
    if (n < 0 || d_model <= 0 || vocab <= 0) return agpt_set_error(AGPT_E_ARG, "embedding_grad_workspace_bytes: bad argument");
    return (int64_t)embedding_blocks(n) * vocab * d_model * 4;
}

extern "C" int agpt_b200_embedding_grad(const float *d_grad, const int32_t *d_ids, float *d_emb_grad, int64_t n, int d_model, int vocab,
                                        int accumulate, void *d_workspace, int64_t workspace_bytes, void *stream) {
    if (!d_grad || !d_ids || !d_emb_grad || n < 0 || d_model <= 0 || vocab <= 0)
        return agpt_set_error(AGPT_E_ARG, "embedding_grad: bad argument");
    const size_t smem = (size_t)vocab * 128 * 4;
    if (smem > 200 * 1024) return agpt_set_error(AGPT_E_LIMIT, "embedding_grad: vocabulary of %d exceeds the shared-memory table (400 symbols)", vocab);
    const int blocks = embedding_blocks(n);
    if (!d_workspace || workspace_bytes < (int64_t)blocks * vocab * d_model * 4)
        return agpt_set_error(AGPT_E_ARG, "embedding_grad: workspace too small (agpt_b200_embedding_grad_workspace_bytes)");
    cudaStream_t st = (cudaStream_t)stream;
    static bool attr_set[64];
    int dev = 0;
    cudaGetDevice(&dev);
    if (dev >= 0 && dev < 64 && !attr_set[dev]) {
        cudaFuncSetAttribute(embedding_grad_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, 200 * 1024);
        attr_set[dev] = true;
    }
    const int64_t chunk = (n + blocks - 1) / blocks;
    dim3 grid(blocks, (d_model + 127) / 128);
    embedding_grad_kernel<<<grid, 128, smem, st>>>(d_grad, d_ids, n, d_model, vocab, chunk, (float *)d_workspace);
    const int64_t vd = (int64_t)vocab * d_model;
    embedding_grad_finish_kernel<<<(unsigned)((vd + 255) / 256), 256, 0, st>>>((const float *)d_workspace, blocks, vd, accumulate, d_emb_grad);
    return launch_status("embedding_grad");
}

// ---- the reference's symbols (void, default stream, 32-bit sizes; errors are kept for agpt_b200_last_error) ---------

extern "C" void cuda_bias_add(float *data, const float *bias, int rows, int cols) { agpt_b200_bias_act(data, bias, data, nullptr, rows, cols, 0, nullptr); }

extern "C" void cuda_fused_bias_relu(const float *input, const float *bias, float *output, float *mask, int rows, int cols) {
    agpt_b200_bias_act(input, bias, output, mask, rows, cols, 1, nullptr);
}

extern "C" void cuda_relu_backward(const float *grad, const float *mask, float *output, int n) { agpt_b200_relu_bwd(grad, mask, output, n, nullptr); }

extern "C" void cuda_softmax_rows(const float *input, float *output, int rows, int cols) { agpt_b200_softmax_rows(input, output, rows, cols, nullptr); }

extern "C" void cuda_softmax_backward(const float *s, const float *ds, float *result, int rows, int cols) {
    agpt_b200_softmax_bwd(s, ds, result, rows, cols, nullptr);
}

extern "C" void cuda_embedding_gather(const float *token_emb, const int *ids, float *output, int seq_len, int d_model) {
    agpt_b200_embedding_gather(token_emb, ids, output, seq_len, d_model, 0, nullptr);
}

extern "C" void cuda_embedding_scatter_add(const float *grad, const int *ids, float *d_token_emb, int seq_len, int d_model) {
    if (!grad || !ids || !d_token_emb || seq_len < 0 || d_model <= 0) {
        agpt_set_error(AGPT_E_ARG, "cuda_embedding_scatter_add: bad argument");
        return;
    }
    if (seq_len == 0) return;
    embedding_scatter_atomic_kernel<<<grid_for((int64_t)seq_len * d_model, 256, 16), 256>>>(grad, ids, d_token_emb, seq_len, d_model);
    launch_status("cuda_embedding_scatter_add");
}
