// Row-wise pieces of the dense step either side of the trie attention: layer norm forward/backward with the
// reference's saved state (normalised rows and 1/std), in float32.
//
// Arithmetic follows the reference's CPU statement of the same routines: mean and biased variance in float32,
// std_inv = 1 / sqrt(var + 1e-5) (src/agpt/incremental_forward.cr:143-163); backward
// dx = (dn - mean(dn) - norm * mean(dn * norm)) * std_inv with dn = grad * gamma, dgamma += sum grad * norm,
// dbeta += sum grad (src/agpt/batched_depth_backward.cr:751-799).  dgamma/dbeta are reduced in a fixed order
// (per-warp, per-block, then block partials in index order): no atomics.
#include <cuda_runtime.h>

#include <cstdint>

#include "../../include/agpt_b200.h"
#include "internal.h"

#define LN_WARPS 8             // warps per block
#define LN_ROWS_PER_WARP 16    // rows a warp walks in the backward kernel
#define LN_MAX_V4 8            // float4 per lane: cols <= 32 * 4 * 8 = 1024

__device__ __forceinline__ float ln_warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

template <int NV>
__global__ void __launch_bounds__(LN_WARPS * 32)
layer_norm_fwd_kernel(const float *__restrict__ x, float *__restrict__ y, float *__restrict__ norm_out,
                      float *__restrict__ std_inv_out, const float *__restrict__ gamma, const float *__restrict__ beta,
                      int64_t rows, int cols) {
    const int64_t r = (int64_t)blockIdx.x * LN_WARPS + (threadIdx.x >> 5);
    if (r >= rows) return;
    const int lane = threadIdx.x & 31, c4n = cols >> 2;
    float4 v[NV];
    float sum = 0.f;
#pragma unroll
    for (int k = 0; k < NV; k++) {
        const int c4 = lane + 32 * k;
        v[k] = c4 < c4n ? __ldcs(reinterpret_cast<const float4 *>(x + r * cols) + c4) : make_float4(0.f, 0.f, 0.f, 0.f);
        sum += (v[k].x + v[k].y) + (v[k].z + v[k].w);
    }
    const float mean = ln_warp_sum(sum) / (float)cols;
    float sq = 0.f;
#pragma unroll
    for (int k = 0; k < NV; k++) {
        if (lane + 32 * k < c4n) {
            v[k].x -= mean; v[k].y -= mean; v[k].z -= mean; v[k].w -= mean;
            sq += (v[k].x * v[k].x + v[k].y * v[k].y) + (v[k].z * v[k].z + v[k].w * v[k].w);
        }
    }
    const float var = ln_warp_sum(sq) / (float)cols;
    const float sinv = 1.0f / sqrtf(var + 1e-5f);
#pragma unroll
    for (int k = 0; k < NV; k++) {
        const int c4 = lane + 32 * k;
        if (c4 >= c4n) continue;
        const float4 g = __ldg(reinterpret_cast<const float4 *>(gamma) + c4), b = __ldg(reinterpret_cast<const float4 *>(beta) + c4);
        const float4 nrm = make_float4(v[k].x * sinv, v[k].y * sinv, v[k].z * sinv, v[k].w * sinv);
        if (norm_out) reinterpret_cast<float4 *>(norm_out + r * cols)[c4] = nrm;
        reinterpret_cast<float4 *>(y + r * cols)[c4] = make_float4(nrm.x * g.x + b.x, nrm.y * g.y + b.y, nrm.z * g.z + b.z, nrm.w * g.w + b.w);
    }
    if (lane == 0 && std_inv_out) std_inv_out[r] = sinv;
}

// dx for LN_ROWS_PER_WARP rows per warp, and the block's partial column sums of grad*norm and grad.
template <int NV>
__global__ void __launch_bounds__(LN_WARPS * 32)
layer_norm_bwd_kernel(const float *grad, const float *__restrict__ norm, const float *__restrict__ std_inv,
                      const float *__restrict__ gamma, const float *add, float *dx, float *__restrict__ partial, int64_t rows,
                      int cols) {
    extern __shared__ float s_part[];      // [LN_WARPS][2][cols]
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, c4n = cols >> 2;
    float4 gam[NV], ag[NV], ab[NV];
#pragma unroll
    for (int k = 0; k < NV; k++) {
        const int c4 = lane + 32 * k;
        gam[k] = c4 < c4n ? __ldg(reinterpret_cast<const float4 *>(gamma) + c4) : make_float4(0.f, 0.f, 0.f, 0.f);
        ag[k] = make_float4(0.f, 0.f, 0.f, 0.f); ab[k] = ag[k];
    }
    const int64_t r_begin = ((int64_t)blockIdx.x * LN_WARPS + warp) * LN_ROWS_PER_WARP;
    for (int64_t r = r_begin; r < r_begin + LN_ROWS_PER_WARP && r < rows; r++) {
        float4 g[NV], nm[NV];
        float s1 = 0.f, s2 = 0.f;
#pragma unroll
        for (int k = 0; k < NV; k++) {
            const int c4 = lane + 32 * k;
            if (c4 < c4n) {
                g[k] = __ldcs(reinterpret_cast<const float4 *>(grad + r * cols) + c4);
                nm[k] = __ldcs(reinterpret_cast<const float4 *>(norm + r * cols) + c4);
            } else { g[k] = make_float4(0.f, 0.f, 0.f, 0.f); nm[k] = g[k]; }
            ag[k].x += g[k].x * nm[k].x; ag[k].y += g[k].y * nm[k].y; ag[k].z += g[k].z * nm[k].z; ag[k].w += g[k].w * nm[k].w;
            ab[k].x += g[k].x; ab[k].y += g[k].y; ab[k].z += g[k].z; ab[k].w += g[k].w;
            g[k].x *= gam[k].x; g[k].y *= gam[k].y; g[k].z *= gam[k].z; g[k].w *= gam[k].w;          // dn
            s1 += (g[k].x + g[k].y) + (g[k].z + g[k].w);
            s2 += (g[k].x * nm[k].x + g[k].y * nm[k].y) + (g[k].z * nm[k].z + g[k].w * nm[k].w);
        }
        const float m1 = ln_warp_sum(s1) / (float)cols, m2 = ln_warp_sum(s2) / (float)cols;
        const float sinv = std_inv[r];
#pragma unroll
        for (int k = 0; k < NV; k++) {
            const int c4 = lane + 32 * k;
            if (c4 >= c4n) continue;
            // the gradient that reaches the same rows by the residual path (may be dx itself: read before written)
            const float4 a = add ? __ldcs(reinterpret_cast<const float4 *>(add + r * cols) + c4) : make_float4(0.f, 0.f, 0.f, 0.f);
            reinterpret_cast<float4 *>(dx + r * cols)[c4] =
                make_float4((g[k].x - m1 - nm[k].x * m2) * sinv + a.x, (g[k].y - m1 - nm[k].y * m2) * sinv + a.y,
                            (g[k].z - m1 - nm[k].z * m2) * sinv + a.z, (g[k].w - m1 - nm[k].w * m2) * sinv + a.w);
        }
    }
    // warps -> block, in warp order
#pragma unroll
    for (int k = 0; k < NV; k++) {
        const int c4 = lane + 32 * k;
        if (c4 >= c4n) continue;
        reinterpret_cast<float4 *>(s_part + (size_t)(warp * 2) * cols)[c4] = ag[k];
        reinterpret_cast<float4 *>(s_part + (size_t)(warp * 2 + 1) * cols)[c4] = ab[k];
    }
    __syncthreads();
    for (int c = threadIdx.x; c < 2 * cols; c += LN_WARPS * 32) {
        const int which = c / cols, col = c % cols;
        float s = 0.f;
#pragma unroll
        for (int w = 0; w < LN_WARPS; w++) s += s_part[(size_t)(w * 2 + which) * cols + col];
        partial[(size_t)blockIdx.x * 2 * cols + c] = s;
    }
}

// dgamma[c] += sum over blocks (in order) of partial[b][0][c]; dbeta likewise.  Each thread walks the blocks
// with a fixed stride and the strided sums are added in thread order.
__global__ void __launch_bounds__(256)
layer_norm_bwd_finish_kernel(const float *__restrict__ partial, float *__restrict__ dgamma, float *__restrict__ dbeta,
                             int64_t n_blocks, int cols) {
    __shared__ float s_acc[256];
    const int c = blockIdx.x;               // column of [2][cols]
    float s = 0.f;
    for (int64_t b = threadIdx.x; b < n_blocks; b += 256) s += partial[(size_t)b * 2 * cols + c];
    s_acc[threadIdx.x] = s;
    __syncthreads();
    for (int off = 128; off > 0; off >>= 1) {
        if (threadIdx.x < off) s_acc[threadIdx.x] += s_acc[threadIdx.x + off];
        __syncthreads();
    }
    if (threadIdx.x == 0) {
        if (c < cols) dgamma[c] += s_acc[0];
        else dbeta[c - cols] += s_acc[0];
    }
}

static int ln_status(const char *what) {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return agpt_set_error(AGPT_E_CUDA, "%s launch: %s", what, cudaGetErrorString(e));
    return AGPT_OK;
}

static int ln_check(int64_t rows, int cols, const char *who) {
    if (rows < 0 || cols < 4 || cols % 4 || cols > 32 * 4 * LN_MAX_V4)
        return agpt_set_error(AGPT_E_ARG, "%s: cols must be a multiple of 4 in [4, %d]", who, 32 * 4 * LN_MAX_V4);
    return AGPT_OK;
}

extern "C" int64_t agpt_b200_layer_norm_bwd_workspace_bytes(int64_t rows, int cols) {
    const int64_t n_blocks = (rows + LN_WARPS * LN_ROWS_PER_WARP - 1) / (LN_WARPS * LN_ROWS_PER_WARP);
    return (n_blocks > 0 ? n_blocks : 1) * 2 * (int64_t)cols * (int64_t)sizeof(float);
}

extern "C" int agpt_b200_layer_norm_fwd(const float *d_x, float *d_y, float *d_norm, float *d_std_inv, const float *d_gamma,
                                        const float *d_beta, int64_t rows, int cols, void *stream) {
    int rc = ln_check(rows, cols, "layer_norm_fwd");
    if (rc) return rc;
    if (!d_x || !d_y || !d_gamma || !d_beta) return agpt_set_error(AGPT_E_ARG, "layer_norm_fwd: null buffer");
    if (rows == 0) return AGPT_OK;
    const unsigned blocks = (unsigned)((rows + LN_WARPS - 1) / LN_WARPS);
    const int nv = (cols / 4 + 31) / 32;
    cudaStream_t st = (cudaStream_t)stream;
#define LN_FWD(NV) layer_norm_fwd_kernel<NV><<<blocks, LN_WARPS * 32, 0, st>>>(d_x, d_y, d_norm, d_std_inv, d_gamma, d_beta, rows, cols)
    if (nv <= 1) LN_FWD(1); else if (nv <= 2) LN_FWD(2); else if (nv <= 4) LN_FWD(4); else LN_FWD(8);
#undef LN_FWD
    return ln_status("layer_norm_fwd");
}

extern "C" int agpt_b200_layer_norm_bwd(const float *d_grad, const float *d_norm, const float *d_std_inv, const float *d_gamma,
                                        float *d_dx, float *d_dgamma, float *d_dbeta, int64_t rows, int cols, void *d_workspace,
                                        int64_t workspace_bytes, void *stream) {
    return agpt_b200_layer_norm_bwd_add(d_grad, d_norm, d_std_inv, d_gamma, nullptr, d_dx, d_dgamma, d_dbeta, rows, cols, d_workspace,
                                        workspace_bytes, stream);
}

extern "C" int agpt_b200_layer_norm_bwd_add(const float *d_grad, const float *d_norm, const float *d_std_inv, const float *d_gamma,
                                            const float *d_add, float *d_dx, float *d_dgamma, float *d_dbeta, int64_t rows, int cols,
                                            void *d_workspace, int64_t workspace_bytes, void *stream) {
    int rc = ln_check(rows, cols, "layer_norm_bwd");
    if (rc) return rc;
    if (!d_grad || !d_norm || !d_std_inv || !d_gamma || !d_dx || !d_dgamma || !d_dbeta || !d_workspace)
        return agpt_set_error(AGPT_E_ARG, "layer_norm_bwd: null buffer");
    if (workspace_bytes < agpt_b200_layer_norm_bwd_workspace_bytes(rows, cols))
        return agpt_set_error(AGPT_E_ARG, "layer_norm_bwd: workspace too small");
    if (rows == 0) return AGPT_OK;
    const int64_t n_blocks = (rows + LN_WARPS * LN_ROWS_PER_WARP - 1) / (LN_WARPS * LN_ROWS_PER_WARP);
    const int nv = (cols / 4 + 31) / 32;
    const size_t smem = (size_t)LN_WARPS * 2 * cols * sizeof(float);
    cudaStream_t st = (cudaStream_t)stream;
    float *partial = (float *)d_workspace;
#define LN_BWD(NV)                                                                                                     \
    do {                                                                                                               \
        cudaError_t e_ = cudaFuncSetAttribute(layer_norm_bwd_kernel<NV>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
        if (e_ != cudaSuccess) return agpt_set_error(AGPT_E_CUDA, "layer_norm_bwd: %s", cudaGetErrorString(e_));       \
        layer_norm_bwd_kernel<NV><<<(unsigned)n_blocks, LN_WARPS * 32, smem, st>>>(d_grad, d_norm, d_std_inv, d_gamma, d_add, d_dx, partial, rows, cols); \
    } while (0)
    if (nv <= 1) LN_BWD(1); else if (nv <= 2) LN_BWD(2); else if (nv <= 4) LN_BWD(4); else LN_BWD(8);
#undef LN_BWD
    if ((rc = ln_status("layer_norm_bwd"))) return rc;
    layer_norm_bwd_finish_kernel<<<(unsigned)(2 * cols), 256, 0, st>>>(partial, d_dgamma, d_dbeta, n_blocks, cols);
    return ln_status("layer_norm_bwd_finish");
}

// ---- legacy symbols (default stream; the backward's scratch is a per-device buffer the library keeps) ----
static void *g_ln_scratch[64];
static int64_t g_ln_scratch_bytes[64];

extern "C" void cuda_layer_norm_forward(const float *input, float *output, float *norm_out, float *std_inv_out,
                                        const float *gamma, const float *beta, int rows, int cols) {
    agpt_b200_layer_norm_fwd(input, output, norm_out, std_inv_out, gamma, beta, rows, cols, nullptr);
}

extern "C" void cuda_layer_norm_backward(const float *grad, const float *norm, const float *std_inv, const float *gamma,
                                         float *dx, float *dgamma, float *dbeta, int rows, int cols) {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) { agpt_set_error(AGPT_E_CUDA, "cuda_layer_norm_backward: no device"); return; }
    const int64_t need = agpt_b200_layer_norm_bwd_workspace_bytes(rows, cols);
    if (g_ln_scratch_bytes[dev] < need) {
        if (g_ln_scratch[dev]) cudaFree(g_ln_scratch[dev]);
        g_ln_scratch[dev] = nullptr; g_ln_scratch_bytes[dev] = 0;
        if (cudaMalloc(&g_ln_scratch[dev], (size_t)need) != cudaSuccess) { agpt_set_error(AGPT_E_NOMEM, "cuda_layer_norm_backward: scratch"); return; }
        g_ln_scratch_bytes[dev] = need;
    }
    agpt_b200_layer_norm_bwd(grad, norm, std_inv, gamma, dx, dgamma, dbeta, rows, cols, g_ln_scratch[dev], g_ln_scratch_bytes[dev], nullptr);
}
