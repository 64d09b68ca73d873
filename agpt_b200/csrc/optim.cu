// Optimizer step over the flat parameter buffer: gradient clipping by global norm, the update rule (SGD, momentum,
// RMSProp, Adam) and decoupled weight decay.  Replaces the kernel dependency the reference declares at
// src/cuda/agpt_train.cu:64-72 (cuda_adam_bulk, cuda_sgd_bulk, cuda_momentum_bulk, cuda_rmsprop_bulk,
// cuda_weight_decay, cuda_grad_clip_by_norm) and calls in this order at :5135-5162: clip, update, decay.  The
// dependency's source is not part of the reference, so the rules are the textbook ones, fixed here:
//   sgd       p -= lr * g
//   momentum  m = beta * m + g;                       p -= lr * m
//   rmsprop   s = beta * s + (1 - beta) * g^2;        p -= lr * g / (sqrt(s) + eps)
//   adam      m = b1 * m + (1 - b1) * g;  v = b2 * v + (1 - b2) * g^2;
//             p -= lr * (m / (1 - b1^t)) / (sqrt(v / (1 - b2^t)) + eps)         (t counts from 1)
//   decay     p -= lr * wd * p                          (after the update)
//   clip      g *= max_norm / ||g||_2  when ||g||_2 > max_norm
// The native entry point does all of it in two launches (norm partials, then one pass over params/grads/state that
// also clears the gradients when asked); the norm is a two-level sum in a fixed order, so steps repeat bit for bit.
#include <cuda_runtime.h>

#include <cmath>
#include <cstdint>

#include "../../include/agpt_b200.h"
#include "internal.h"

namespace {

constexpr int NORM_BLOCKS_MAX = 1024;

int launch_status(const char *who) {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return agpt_set_error(AGPT_E_CUDA, "%s: %s", who, cudaGetErrorString(e));
    return AGPT_OK;
}

int norm_blocks(int64_t n, int cap) {
    int64_t b = (n + 255) / 256;                      // never more than the reference's ceil(n / 256) partials
    if (b > cap) b = cap;
    return (int)(b < 1 ? 1 : b);
}

// partial[b] = sum of g^2 over the block's contiguous slice
__global__ void __launch_bounds__(256) sq_norm_partial_kernel(const float *__restrict__ g, int64_t n, float *__restrict__ partial) {
    __shared__ float s[256];
    const int64_t per = (n + gridDim.x - 1) / gridDim.x;
    const int64_t a = (int64_t)blockIdx.x * per, b = (a + per < n) ? a + per : n;
    float t = 0.f;
    for (int64_t i = a + threadIdx.x; i < b; i += 256) t += g[i] * g[i];
    s[threadIdx.x] = t;
    __syncthreads();
    for (int k = 128; k > 0; k >>= 1) {
        if (threadIdx.x < k) s[threadIdx.x] += s[threadIdx.x + k];
        __syncthreads();
    }
    if (threadIdx.x == 0) partial[blockIdx.x] = s[0];
}

// every thread adds the partials in the same order: all blocks agree on the norm without another launch
__device__ float norm_from_partials(const float *__restrict__ partial, int blocks) {
    float t = 0.f;
    for (int b = 0; b < blocks; b++) t += partial[b];
    return sqrtf(t);
}

__global__ void __launch_bounds__(256) clip_scale_kernel(float *__restrict__ g, int64_t n, float max_norm, const float *__restrict__ partial,
                                                          int blocks, float *__restrict__ norm_out) {
    const float norm = norm_from_partials(partial, blocks);
    if (norm_out && blockIdx.x == 0 && threadIdx.x == 0) norm_out[0] = norm;
    if (!(norm > max_norm)) return;
    const float scale = max_norm / norm;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) g[i] *= scale;
}

struct StepArgs {
    float lr, beta1, beta2, eps, bc1, bc2, weight_decay, clip_norm;
    int kind, zero_grads, norm_blocks;
};

template <int KIND>
__device__ __forceinline__ float update(float p, float g, float *m, float *v, int64_t i, const StepArgs &a) {
    if (KIND == AGPT_OPT_SGD) {
        p -= a.lr * g;
    } else if (KIND == AGPT_OPT_MOMENTUM) {
        float mi = a.beta1 * m[i] + g;
        m[i] = mi;
        p -= a.lr * mi;
    } else if (KIND == AGPT_OPT_RMSPROP) {
        float si = a.beta2 * v[i] + (1.f - a.beta2) * g * g;
        v[i] = si;
        p -= a.lr * g / (sqrtf(si) + a.eps);
    } else {
        float mi = a.beta1 * m[i] + (1.f - a.beta1) * g;
        float vi = a.beta2 * v[i] + (1.f - a.beta2) * g * g;
        m[i] = mi;
        v[i] = vi;
        p -= a.lr * (mi / a.bc1) / (sqrtf(vi / a.bc2) + a.eps);
    }
    return p;
}

template <int KIND>
__global__ void __launch_bounds__(256) step_kernel(float *__restrict__ p, float *__restrict__ g, float *__restrict__ m, float *__restrict__ v,
                                                    int64_t n, StepArgs a, const float *__restrict__ partial, float *__restrict__ norm_out) {
    float scale = 1.f;
    if (a.clip_norm > 0.f) {
        const float norm = norm_from_partials(partial, a.norm_blocks);
        if (norm_out && blockIdx.x == 0 && threadIdx.x == 0) norm_out[0] = norm;
        if (norm > a.clip_norm) scale = a.clip_norm / norm;
    }
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) {
        float gi = g[i] * scale;
        float pi = update<KIND>(p[i], gi, m, v, i, a);
        if (a.weight_decay > 0.f) pi -= a.lr * a.weight_decay * pi;
        p[i] = pi;
        if (a.zero_grads) g[i] = 0.f;
    }
}

unsigned step_grid(int64_t n) {
    int64_t b = (n + 255) / 256;
    return (unsigned)(b < 1 ? 1 : (b < 148 * 8 ? b : 148 * 8));
}

int run_step(int kind, float *p, float *g, float *m, float *v, int64_t n, const StepArgs &a, const float *partial, float *norm_out,
             cudaStream_t st) {
    unsigned grid = step_grid(n);
    switch (kind) {
        case AGPT_OPT_SGD: step_kernel<AGPT_OPT_SGD><<<grid, 256, 0, st>>>(p, g, m, v, n, a, partial, norm_out); break;
        case AGPT_OPT_MOMENTUM: step_kernel<AGPT_OPT_MOMENTUM><<<grid, 256, 0, st>>>(p, g, m, v, n, a, partial, norm_out); break;
        case AGPT_OPT_RMSPROP: step_kernel<AGPT_OPT_RMSPROP><<<grid, 256, 0, st>>>(p, g, m, v, n, a, partial, norm_out); break;
        case AGPT_OPT_ADAM: step_kernel<AGPT_OPT_ADAM><<<grid, 256, 0, st>>>(p, g, m, v, n, a, partial, norm_out); break;
        default: return agpt_set_error(AGPT_E_ARG, "optimizer_step: unknown optimizer kind %d", kind);
    }
    return launch_status("optimizer_step");
}

__global__ void __launch_bounds__(256) weight_decay_kernel(float *__restrict__ p, float f, int64_t n) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (int64_t)gridDim.x * blockDim.x) p[i] -= f * p[i];
}

}  // namespace

extern "C" int64_t agpt_b200_optimizer_scratch_bytes(void) { return (int64_t)(NORM_BLOCKS_MAX + 1) * 4; }

extern "C" int agpt_b200_optimizer_step(int kind, float *d_params, float *d_grads, float *d_m, float *d_v, int64_t n, float lr, float beta1,
                                        float beta2, float eps, int t, float weight_decay, float clip_norm, int zero_grads,
                                        void *d_scratch, void *stream) {
    if (!d_params || !d_grads || n < 0) return agpt_set_error(AGPT_E_ARG, "optimizer_step: bad argument");
    if ((kind == AGPT_OPT_MOMENTUM || kind == AGPT_OPT_ADAM) && !d_m) return agpt_set_error(AGPT_E_ARG, "optimizer_step: first-moment buffer missing");
    if ((kind == AGPT_OPT_RMSPROP || kind == AGPT_OPT_ADAM) && !d_v) return agpt_set_error(AGPT_E_ARG, "optimizer_step: second-moment buffer missing");
    if (kind == AGPT_OPT_ADAM && t < 1) return agpt_set_error(AGPT_E_ARG, "optimizer_step: Adam's step counter starts at 1");
    if (clip_norm > 0.f && !d_scratch) return agpt_set_error(AGPT_E_ARG, "optimizer_step: clipping needs the scratch buffer");
    if (n == 0) return AGPT_OK;
    cudaStream_t st = (cudaStream_t)stream;
    StepArgs a;
    a.lr = lr; a.beta1 = beta1; a.beta2 = beta2; a.eps = eps; a.weight_decay = weight_decay; a.clip_norm = clip_norm;
    a.bc1 = kind == AGPT_OPT_ADAM ? 1.f - powf(beta1, (float)t) : 1.f;
    a.bc2 = kind == AGPT_OPT_ADAM ? 1.f - powf(beta2, (float)t) : 1.f;
    a.kind = kind; a.zero_grads = zero_grads; a.norm_blocks = 0;
    float *partial = (float *)d_scratch;
    if (clip_norm > 0.f) {
        a.norm_blocks = norm_blocks(n, NORM_BLOCKS_MAX);
        sq_norm_partial_kernel<<<a.norm_blocks, 256, 0, st>>>(d_grads, n, partial);
    }
    return run_step(kind, d_params, d_grads, d_m, d_v, n, a, partial, partial ? partial + NORM_BLOCKS_MAX : nullptr, st);
}

// ---- the reference's symbols (void, default stream, 32-bit sizes) -------------------------------------------------

static void legacy_step(int kind, float *p, float *g, float *m, float *v, float lr, float b1, float b2, float eps, int t, int n) {
    agpt_b200_optimizer_step(kind, p, g, m, v, n, lr, b1, b2, eps, t, 0.f, 0.f, 0, nullptr, nullptr);
}

extern "C" void cuda_adam_bulk(float *params, float *grads, float *m, float *v, float lr, float beta1, float beta2, float eps, int t, int n) {
    legacy_step(AGPT_OPT_ADAM, params, grads, m, v, lr, beta1, beta2, eps, t, n);
}

extern "C" void cuda_sgd_bulk(float *params, float *grads, float lr, int n) { legacy_step(AGPT_OPT_SGD, params, grads, nullptr, nullptr, lr, 0.f, 0.f, 0.f, 1, n); }

extern "C" void cuda_momentum_bulk(float *params, float *grads, float *m, float lr, float beta, int n) {
    legacy_step(AGPT_OPT_MOMENTUM, params, grads, m, nullptr, lr, beta, 0.f, 0.f, 1, n);
}

extern "C" void cuda_rmsprop_bulk(float *params, float *grads, float *s, float lr, float beta, float eps, int n) {
    legacy_step(AGPT_OPT_RMSPROP, params, grads, nullptr, s, lr, 0.f, beta, eps, 1, n);
}

extern "C" void cuda_weight_decay(float *params, float lr, float wd, int n) {
    if (!params || n < 0) {
        agpt_set_error(AGPT_E_ARG, "cuda_weight_decay: bad argument");
        return;
    }
    if (n == 0) return;
    weight_decay_kernel<<<step_grid(n), 256>>>(params, lr * wd, n);
    launch_status("cuda_weight_decay");
}

// partials_scratch holds ceil(n / 256) floats in the reference (src/cuda/agpt_train.cu:3334-3338); at most that many are used
extern "C" void cuda_grad_clip_by_norm(float *grads, float max_norm, int n, float *partials_scratch, float *norm_scratch) {
    if (!grads || !partials_scratch || n < 0) {
        agpt_set_error(AGPT_E_ARG, "cuda_grad_clip_by_norm: bad argument");
        return;
    }
    if (n == 0) return;
    const int blocks = norm_blocks(n, NORM_BLOCKS_MAX);
    sq_norm_partial_kernel<<<blocks, 256>>>(grads, n, partials_scratch);
    clip_scale_kernel<<<step_grid(n), 256>>>(grads, n, max_norm, partials_scratch, blocks, norm_scratch);
    launch_status("cuda_grad_clip_by_norm");
}
