// CUDA side of libagpt_b200 (sm_100a): trie-scoped attention forward/backward over a
// depth-first KV store, the deterministic dK/dV reduction, the per-query loss, RoPE, and the
// legacy packed-prefix kernels.
//
// Layout.  Activations are row-major [n, H*hd] in the plan's depth-first order, so a node's
// subtree is a contiguous row interval and the keys a tile of M consecutive queries can attend
// are exactly: the ancestor chain of the tile's first query (shared by the whole tile, listed in
// chain_ids) plus the tile's own rows.  Key a is attended by query i iff a <= i < sub_end[a].
#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>

#include <algorithm>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <vector>

#include "../../include/agpt_b200.h"
#include "internal.h"

#define CUDA_TRY(x)                                                                              \
    do {                                                                                         \
        cudaError_t e_ = (x);                                                                    \
        if (e_ != cudaSuccess) return agpt_set_error(AGPT_E_CUDA, "%s: %s", #x, cudaGetErrorString(e_)); \
    } while (0)

static inline int launch_status(const char *what) {
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return agpt_set_error(AGPT_E_CUDA, "%s launch: %s", what, cudaGetErrorString(e));
    return AGPT_OK;
}

#define AGPT_MAX_DEVICES 64
// Raise a kernel's dynamic shared-memory limit once per device (the attribute belongs to the context's copy of the
// function, so it is set again on every device a plan is used on, but not on every launch).
template <typename KernelT>
static int allow_dynamic_smem(KernelT kernel, size_t bytes, size_t *granted /* [AGPT_MAX_DEVICES] */) {
    int dev = 0;
    CUDA_TRY(cudaGetDevice(&dev));
    if (dev < 0 || dev >= AGPT_MAX_DEVICES) return agpt_set_error(AGPT_E_LIMIT, "device index %d beyond %d", dev, AGPT_MAX_DEVICES);
    if (granted[dev] < bytes) {
        CUDA_TRY(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)bytes));
        granted[dev] = bytes;
    }
    return AGPT_OK;
}

// --------------------------------------------------------------------------------------
// plan: device copies
// --------------------------------------------------------------------------------------
template <typename T>
static int upload(T **dst, const std::vector<T> &src) {
    size_t bytes = (src.size() ? src.size() : 1) * sizeof(T);
    CUDA_TRY(cudaMalloc((void **)dst, bytes));
    if (!src.empty()) CUDA_TRY(cudaMemcpy(*dst, src.data(), src.size() * sizeof(T), cudaMemcpyHostToDevice));
    return AGPT_OK;
}

int agpt_plan_upload(agpt_plan *p, int device) {
    CUDA_TRY(cudaSetDevice(device));
    p->device = device;
    int rc;
    if ((rc = upload(&p->d_depth, p->depth))) return rc;
    if ((rc = upload(&p->d_sub_end, p->sub_end))) return rc;
    if ((rc = upload(&p->d_chain_ids, p->chain_ids))) return rc;
    if ((rc = upload(&p->d_chain_end, p->chain_end))) return rc;
    if ((rc = upload(&p->d_chain_off, p->chain_off))) return rc;
    if ((rc = upload(&p->d_item_node, p->item_node))) return rc;
    if ((rc = upload(&p->d_item_t0, p->item_t0))) return rc;
    if ((rc = upload(&p->d_item_t1, p->item_t1))) return rc;
    if ((rc = upload(&p->d_item_slot, p->item_slot))) return rc;
    if ((rc = upload(&p->d_multi_node, p->multi_node))) return rc;
    if ((rc = upload(&p->d_multi_count, p->multi_count))) return rc;
    if ((rc = upload(&p->d_multi_first, p->multi_first))) return rc;
    return AGPT_OK;
}

agpt_plan::~agpt_plan() {
    if (device >= 0) {
        int cur = -1;
        cudaGetDevice(&cur);
        cudaSetDevice(device);
        cudaFree(d_depth); cudaFree(d_sub_end); cudaFree(d_chain_ids); cudaFree(d_chain_end); cudaFree(d_chain_off);
        cudaFree(d_item_node); cudaFree(d_item_t0); cudaFree(d_item_t1); cudaFree(d_item_slot);
        cudaFree(d_multi_node); cudaFree(d_multi_count); cudaFree(d_multi_first);
        cudaFree(host_arena);
        if (host_fix) cudaFreeHost(host_fix);
        for (void *e : host_events) cudaEventDestroy((cudaEvent_t)e);
        for (void *st : host_streams) if (st) cudaStreamDestroy((cudaStream_t)st);
        if (cur >= 0) cudaSetDevice(cur);
    }
}

extern "C" void agpt_b200_plan_destroy(agpt_plan *p) { delete p; }

// --------------------------------------------------------------------------------------
// small helpers
// --------------------------------------------------------------------------------------
// Which (key, query) pairs feed dK/dV (dQ always takes every attended key).  A pair with key id a and query id i
// (a <= i) is kept iff a >= first(i): first(i) = -inf keeps all (full: a node's dK/dV sum over the node itself and all
// its descendants), first(i) = i keeps the query's own key only (local depth), first(i) = edge_first[i] keeps the keys
// on the query's own radix edge.
struct BwdMask {
    int mode;                       // AGPT_GRAD_*
    const int32_t *edge_first;      // [n] depth-first position of the first char of each position's radix edge (mode 2)
};
__device__ __forceinline__ int bwd_first_key(const BwdMask &mk, int i, int n) {
    if (mk.mode == AGPT_GRAD_FULL || i >= n) return -0x7fffffff - 1;
    return mk.mode == AGPT_GRAD_LOCAL_DEPTH ? i : __ldg(mk.edge_first + i);
}

#define KC 32            // keys staged per chunk
#define LOG2E 1.4426950408889634f
#define LN2 0.6931471805599453f

__device__ __forceinline__ float4 ld4(const float *p) { return __ldg(reinterpret_cast<const float4 *>(p)); }
__device__ __forceinline__ float4 ld4(const __nv_bfloat16 *p) {
    uint2 raw = __ldg(reinterpret_cast<const uint2 *>(p));
    float4 r;
    r.x = __uint_as_float(raw.x << 16); r.y = __uint_as_float(raw.x & 0xffff0000u);
    r.z = __uint_as_float(raw.y << 16); r.w = __uint_as_float(raw.y & 0xffff0000u);
    return r;
}

// Stage the id, subtree end and K/V rows of keys [kc, kc+cnt) of a tile into shared memory.
template <int HD, int NT, typename KVT>
__device__ __forceinline__ void stage_keys(const KVT *__restrict__ K, const KVT *__restrict__ V,
                                           const int32_t *__restrict__ sub_end, const int32_t *__restrict__ chain,
                                           int p, int i0, int kc, int cnt, int D, int hoff, int *s_kid, int *s_kend,
                                           float (*sK)[HD + 4], float (*sV)[HD + 4]) {
    const int tid = threadIdx.x;
    if (tid < KC) {
        int kk = kc + tid, kid = -1, kend = 0;
        if (tid < cnt) { kid = kk < p ? chain[kk] : i0 + (kk - p); kend = sub_end[kid]; }
        s_kid[tid] = kid; s_kend[tid] = kend;
    }
    __syncthreads();
    constexpr int C4 = HD / 4;
    for (int idx = tid; idx < cnt * C4; idx += NT) {
        int r = idx / C4, c = idx % C4;
        int64_t base = (int64_t)s_kid[r] * D + hoff + c * 4;
        *reinterpret_cast<float4 *>(&sK[r][c * 4]) = ld4(K + base);
        *reinterpret_cast<float4 *>(&sV[r][c * 4]) = ld4(V + base);
    }
    __syncthreads();
}

// --------------------------------------------------------------------------------------
// forward: one thread per (query, head); keys broadcast from shared memory
// --------------------------------------------------------------------------------------
template <int HD, int M, typename KVT>
__global__ void __launch_bounds__(M) attn_fwd_kernel(const float *__restrict__ Q, const KVT *__restrict__ K,
                                                     const KVT *__restrict__ V, float *__restrict__ O,
                                                     float *__restrict__ LSE, const int32_t *__restrict__ sub_end,
                                                     const int64_t *__restrict__ chain_off,
                                                     const int32_t *__restrict__ chain_ids, int n, int H, float scale, int tile0) {
    __shared__ __align__(16) float sK[KC][HD + 4];
    __shared__ __align__(16) float sV[KC][HD + 4];
    __shared__ int s_kid[KC], s_kend[KC];
    const int t = blockIdx.x + tile0, h = blockIdx.y, tid = threadIdx.x;
    const int D = H * HD, hoff = h * HD;
    const int i0 = t * M, i = i0 + tid;
    const bool active = i < n;
    const int64_t coff = chain_off[t];
    const int p = (int)(chain_off[t + 1] - coff);
    const int nkeys = p + min(M, n - i0);
    const int32_t *chain = chain_ids + coff;

    float q[HD], acc[HD];
    const float qs = scale * LOG2E;
#pragma unroll
    for (int c = 0; c < HD / 4; c++) {
        float4 x = active ? ld4(Q + (int64_t)i * D + hoff + c * 4) : make_float4(0.f, 0.f, 0.f, 0.f);
        q[4 * c] = x.x * qs; q[4 * c + 1] = x.y * qs; q[4 * c + 2] = x.z * qs; q[4 * c + 3] = x.w * qs;
        acc[4 * c] = acc[4 * c + 1] = acc[4 * c + 2] = acc[4 * c + 3] = 0.f;
    }
    float m = -INFINITY, l = 0.f;

    for (int kc = 0; kc < nkeys; kc += KC) {
        const int cnt = min(KC, nkeys - kc);
        __syncthreads();
        stage_keys<HD, M, KVT>(K, V, sub_end, chain, p, i0, kc, cnt, D, hoff, s_kid, s_kend, sK, sV);
        for (int j0 = 0; j0 < cnt; j0 += 4) {
            bool vld[4];
            bool anyv = false;
#pragma unroll
            for (int jj = 0; jj < 4; jj++) {
                int j = j0 + jj;
                vld[jj] = active && j < cnt && s_kid[j] <= i && i < s_kend[j];
                anyv |= vld[jj];
            }
            if (!__any_sync(0xffffffffu, anyv)) continue;
            float s[4];
#pragma unroll
            for (int jj = 0; jj < 4; jj++) {
                int j = min(j0 + jj, cnt - 1);
                float d0 = 0.f, d1 = 0.f;
#pragma unroll
                for (int c = 0; c < HD / 4; c++) {
                    float4 kk = *reinterpret_cast<const float4 *>(&sK[j][c * 4]);
                    d0 = fmaf(q[4 * c], kk.x, d0); d1 = fmaf(q[4 * c + 1], kk.y, d1);
                    d0 = fmaf(q[4 * c + 2], kk.z, d0); d1 = fmaf(q[4 * c + 3], kk.w, d1);
                }
                s[jj] = vld[jj] ? d0 + d1 : -INFINITY;
            }
            float mx = fmaxf(fmaxf(s[0], s[1]), fmaxf(s[2], s[3]));
            float mn = fmaxf(m, mx);
            float mu = mn == -INFINITY ? 0.f : mn;
            float corr = exp2f(m - mu);
            m = mn;
            l *= corr;
#pragma unroll
            for (int d = 0; d < HD; d++) acc[d] *= corr;
#pragma unroll
            for (int jj = 0; jj < 4; jj++) {
                int j = min(j0 + jj, cnt - 1);
                float w = exp2f(s[jj] - mu);
                l += w;
#pragma unroll
                for (int c = 0; c < HD / 4; c++) {
                    float4 vv = *reinterpret_cast<const float4 *>(&sV[j][c * 4]);
                    acc[4 * c] = fmaf(w, vv.x, acc[4 * c]); acc[4 * c + 1] = fmaf(w, vv.y, acc[4 * c + 1]);
                    acc[4 * c + 2] = fmaf(w, vv.z, acc[4 * c + 2]); acc[4 * c + 3] = fmaf(w, vv.w, acc[4 * c + 3]);
                }
            }
        }
    }
    if (active) {
        float inv = 1.0f / l;
#pragma unroll
        for (int c = 0; c < HD / 4; c++)
            *reinterpret_cast<float4 *>(O + (int64_t)i * D + hoff + c * 4) =
                make_float4(acc[4 * c] * inv, acc[4 * c + 1] * inv, acc[4 * c + 2] * inv, acc[4 * c + 3] * inv);
        LSE[(int64_t)i * H + h] = (m + log2f(l)) * LN2;
    }
}

// --------------------------------------------------------------------------------------
// forward on the tensor cores: mma.sync m16n8k8 TF32 with error compensation.
//
// A tile of 64 depth-first-consecutive queries against (chain + tile) keys is a dense 64 x (p + 64)
// problem with an interval mask, so QK^T and PV run as 16x8x8 MMAs: 4 warps x 16 query rows, key blocks of
// 8.  float32 parity needs more than TF32's 10-bit mantissa, so every operand is split x = hi + lo
// (hi = x rounded to TF32) and each product is hi*hi + lo*hi + hi*lo (the dropped lo*lo term is ~2^-22
// relative).  A bf16 store is exact in TF32, so its lo part is absent and two MMAs suffice.  A warp skips
// every 16x8 block in which none of its queries may attend any of the 8 keys.
// --------------------------------------------------------------------------------------
__device__ __forceinline__ uint32_t tf32_round(float x) {
    uint32_t r;
    asm("cvt.rna.tf32.f32 %0, %1;" : "=r"(r) : "f"(x));
    return r;
}
__device__ __forceinline__ void tf32_split(float x, uint32_t &hi, uint32_t &lo) {
    hi = tf32_round(x);
    lo = __float_as_uint(x - __uint_as_float(hi));
}
__device__ __forceinline__ void mma_tf32(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k8.row.col.f32.tf32.tf32.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

#define MAXKEYS 512      // keys (chain + tile rows) a tile of the tensor-core kernels can hold metadata for

__device__ __forceinline__ void cp_async16(void *smem_dst, const void *gmem_src) {
    unsigned d = (unsigned)__cvta_generic_to_shared(smem_dst);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(gmem_src));
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::); }
__device__ __forceinline__ void cp_async_wait_all() { asm volatile("cp.async.wait_group 0;" ::: "memory"); }

// Id and subtree end of every key of the tile (chain first, then the tile's own rows): one round of
// independent loads (chain_end is precomputed so that no load depends on another).  128 threads.
__device__ __forceinline__ void load_key_meta(const int32_t *__restrict__ sub_end, const int32_t *__restrict__ chain,
                                              const int32_t *__restrict__ chain_end, int p, int i0, int nkeys, int *s_kid,
                                              int *s_kend) {
    for (int j = threadIdx.x; j < nkeys; j += 128) {
        int kid, kend;
        if (j < p) { kid = __ldg(chain + j); kend = __ldg(chain_end + j); }
        else { kid = i0 + (j - p); kend = __ldg(sub_end + kid); }
        s_kid[j] = kid; s_kend[j] = kend;
    }
}

// Shared-memory form of a staged K/V row: float32 rows as they are (padded by 4 floats), bf16 rows as raw
// bf16 (padded by 8 elements) and widened when a fragment is read; both paddings make the MMA fragment reads
// bank-conflict free and keep every row 16-byte aligned for cp.async.
template <typename KVT> struct SmemKV;
template <> struct SmemKV<float> { typedef float elem; static constexpr int PAD = 4; };
template <> struct SmemKV<__nv_bfloat16> { typedef unsigned short elem; static constexpr int PAD = 8; };
__device__ __forceinline__ float kv_f32(float x) { return x; }
__device__ __forceinline__ float kv_f32(unsigned short x) { return __uint_as_float((unsigned)x << 16); }

// Start the copy of keys [kc, kc+cnt) into one shared-memory buffer with cp.async (the copy overlaps the MMAs on
// other buffers).  Rows beyond cnt are zero-filled: they enter MMAs with weight 0.  128 threads; the caller
// waits and synchronises.
template <int HD, typename KVT>
__device__ __forceinline__ void issue_chunk(const KVT *__restrict__ K, const KVT *__restrict__ V, const int *s_kid, int kc,
                                            int cnt, int D, int hoff,
                                            typename SmemKV<KVT>::elem (*sK)[HD + SmemKV<KVT>::PAD],
                                            typename SmemKV<KVT>::elem (*sV)[HD + SmemKV<KVT>::PAD]) {
    constexpr int EPC = 16 / sizeof(KVT);          // elements per 16-byte copy
    constexpr int CPR = HD / EPC;                   // copies per row
    for (int idx = threadIdx.x; idx < KC * CPR; idx += 128) {
        const int r = idx / CPR, c = idx % CPR;
        if (r < cnt) {
            const int64_t base = (int64_t)s_kid[kc + r] * D + hoff + c * EPC;
            cp_async16(&sK[r][c * EPC], K + base);
            cp_async16(&sV[r][c * EPC], V + base);
        } else {
            *reinterpret_cast<uint4 *>(&sK[r][c * EPC]) = make_uint4(0u, 0u, 0u, 0u);
            *reinterpret_cast<uint4 *>(&sV[r][c * EPC]) = make_uint4(0u, 0u, 0u, 0u);
        }
    }
    cp_async_commit();
}

// At head_dim 64 (few warps per SM) the chunked backward computes both 8-key halves of a 16-key block that has any valid
// pair, the half without one included: the masked half costs a few products whose results are exact zeros, and the two
// independent chains of products interleave in one basic block.  Measured on the 4M-node tree with the bf16 store: 25.6 ms
// against 26.8 ms.  (The same in the chunked forward, all four 8-key blocks of a chunk in one basic block, lost: 17.6
// against 14.9 ms with the float32 store, 11.2 against 11.0 ms with bf16.)
#ifndef AGPT_CHUNK_BOTH_MIN_HD
#define AGPT_CHUNK_BOTH_MIN_HD 64
#endif
template <int HD> struct ChunkBothHalves { static constexpr bool value = HD >= AGPT_CHUNK_BOTH_MIN_HD; };

template <int HD> struct FwdMmaStages { static constexpr int value = HD <= 16 ? 4 : 3; };
template <int HD> constexpr size_t fwd_mma_smem_bytes() {
    return (size_t)FwdMmaStages<HD>::value * 2 * KC * (HD + 8) * sizeof(float) + 2 * MAXKEYS * sizeof(int);   // upper bound
}

template <int HD, typename KVT>
__global__ void __launch_bounds__(128) attn_fwd_mma_kernel(const float *__restrict__ Q, const KVT *__restrict__ K,
                                                           const KVT *__restrict__ V, float *__restrict__ O,
                                                           float *__restrict__ LSE, const int32_t *__restrict__ sub_end,
                                                           const int64_t *__restrict__ chain_off,
                                                           const int32_t *__restrict__ chain_ids,
                                                           const int32_t *__restrict__ chain_end_all, int n, int H,
                                                           float scale, int tile0) {
    constexpr int M = 64, KS = HD / 8;
    constexpr bool SPLIT_KV = sizeof(KVT) == 4;
    // NS key chunks are staged per round and consumed without any barrier in between, so the four warps (whose
    // live key blocks differ a lot: later rows attend more of the tile) do not wait for each other per chunk
    constexpr int NS = FwdMmaStages<HD>::value;
    extern __shared__ __align__(16) unsigned char fwd_smem_raw[];
    typedef typename SmemKV<KVT>::elem SE;
    constexpr int SP = HD + SmemKV<KVT>::PAD;
    typedef SE (*KvBuf)[KC][SP];
    KvBuf sKb = reinterpret_cast<KvBuf>(fwd_smem_raw);
    KvBuf sVb = sKb + NS;
    int *s_kid = reinterpret_cast<int *>(sVb + NS), *s_kend = s_kid + MAXKEYS;
    const int t = blockIdx.x + tile0, h = blockIdx.y, tid = threadIdx.x;
    const int warp = tid >> 5, lane = tid & 31, g = lane >> 2, tig = lane & 3;
    const int D = H * HD, hoff = h * HD;
    const int i0 = t * M;
    const int r0 = i0 + warp * 16 + g, r1 = r0 + 8;
    const bool act0 = r0 < n, act1 = r1 < n;
    const int64_t coff = chain_off[t];
    const int p = (int)(chain_off[t + 1] - coff);
    const int nkeys = p + min(M, n - i0);
    const int32_t *chain = chain_ids + coff;
    const float qs = scale * LOG2E;
    load_key_meta(sub_end, chain, chain_end_all + coff, p, i0, nkeys, s_kid, s_kend);
    __syncthreads();
    auto issue_round = [&](int rb) {
#pragma unroll
        for (int st = 0; st < NS; st++) {
            const int kc = rb + st * KC;
            if (kc < nkeys) issue_chunk<HD, KVT>(K, V, s_kid, kc, min(KC, nkeys - kc), D, hoff, sKb[st], sVb[st]);
        }
    };
    issue_round(0);

    uint32_t qh[KS][4], ql[KS][4];
#pragma unroll
    for (int ks = 0; ks < KS; ks++) {
        const int d0 = hoff + ks * 8 + tig;
        float x0 = act0 ? __ldg(Q + (int64_t)r0 * D + d0) * qs : 0.f;
        float x1 = act1 ? __ldg(Q + (int64_t)r1 * D + d0) * qs : 0.f;
        float x2 = act0 ? __ldg(Q + (int64_t)r0 * D + d0 + 4) * qs : 0.f;
        float x3 = act1 ? __ldg(Q + (int64_t)r1 * D + d0 + 4) * qs : 0.f;
        tf32_split(x0, qh[ks][0], ql[ks][0]); tf32_split(x1, qh[ks][1], ql[ks][1]);
        tf32_split(x2, qh[ks][2], ql[ks][2]); tf32_split(x3, qh[ks][3], ql[ks][3]);
    }
    float o[KS][4];
#pragma unroll
    for (int db = 0; db < KS; db++) o[db][0] = o[db][1] = o[db][2] = o[db][3] = 0.f;
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;

    for (int kc = 0; kc < nkeys; kc += KC) {
        const int st = (kc / KC) % NS;
        if (st == 0) {
            if (kc > 0) { __syncthreads(); issue_round(kc); }      // every warp is done with the previous round
            cp_async_wait_all();
            __syncthreads();                                       // this round's chunks have landed
        }
        SE (*sK)[SP] = sKb[st];
        SE (*sV)[SP] = sVb[st];
        float s[KC / 8][4];
        unsigned live = 0;
#pragma unroll
        for (int nb = 0; nb < KC / 8; nb++) {
            const int kA = nb * 8 + 2 * tig;
            const bool inA = kc + kA < nkeys, inB = kc + kA + 1 < nkeys;
            const int kidA = inA ? s_kid[kc + kA] : 0, kendA = inA ? s_kend[kc + kA] : 0;
            const int kidB = inB ? s_kid[kc + kA + 1] : 0, kendB = inB ? s_kend[kc + kA + 1] : 0;
            const bool v0 = act0 && kidA <= r0 && r0 < kendA, v1 = act0 && kidB <= r0 && r0 < kendB;
            const bool v2 = act1 && kidA <= r1 && r1 < kendA, v3 = act1 && kidB <= r1 && r1 < kendB;
            s[nb][0] = s[nb][1] = s[nb][2] = s[nb][3] = -INFINITY;
            if (!__any_sync(0xffffffffu, v0 | v1 | v2 | v3)) continue;
            live |= 1u << nb;
            // the three products of a score accumulate in separate chains (two at head_dim <= 32, where a third
            // accumulator would cost a resident block): dependent MMAs are what a warp waits on here
            float c[4] = {0.f, 0.f, 0.f, 0.f}, cx[4] = {0.f, 0.f, 0.f, 0.f}, cy[4] = {0.f, 0.f, 0.f, 0.f};
#pragma unroll
            for (int ks = 0; ks < KS; ks++) {
                const float b0 = kv_f32(sK[nb * 8 + g][ks * 8 + tig]), b1 = kv_f32(sK[nb * 8 + g][ks * 8 + tig + 4]);
                if (SPLIT_KV) {
                    uint32_t h0, lo0, h1, lo1;
                    tf32_split(b0, h0, lo0); tf32_split(b1, h1, lo1);
                    mma_tf32(c, qh[ks], h0, h1); mma_tf32(cx, ql[ks], h0, h1);
                    if (HD >= 64) mma_tf32(cy, qh[ks], lo0, lo1);
                    else mma_tf32(cx, qh[ks], lo0, lo1);
                } else {
                    // bf16 store: K is exact in TF32 and the store's own rounding (2^-9) dwarfs TF32's (2^-11) on Q,
                    // so one product is enough for the bf16-store tolerance
                    mma_tf32(c, qh[ks], __float_as_uint(b0), __float_as_uint(b1));
                }
            }
            c[0] += cx[0] + cy[0]; c[1] += cx[1] + cy[1]; c[2] += cx[2] + cy[2]; c[3] += cx[3] + cy[3];
            if (v0) s[nb][0] = c[0];
            if (v1) s[nb][1] = c[1];
            if (v2) s[nb][2] = c[2];
            if (v3) s[nb][3] = c[3];
        }
        if (live == 0) continue;                       // warp-uniform
        float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
        for (int nb = 0; nb < KC / 8; nb++) {
            mx0 = fmaxf(mx0, fmaxf(s[nb][0], s[nb][1]));
            mx1 = fmaxf(mx1, fmaxf(s[nb][2], s[nb][3]));
        }
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1)); mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1)); mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
        const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
        const float mu0 = mn0 == -INFINITY ? 0.f : mn0, mu1 = mn1 == -INFINITY ? 0.f : mn1;
        const float corr0 = exp2f(m0 - mu0), corr1 = exp2f(m1 - mu1);
        m0 = mn0; m1 = mn1;
        l0 *= corr0; l1 *= corr1;
#pragma unroll
        for (int db = 0; db < KS; db++) { o[db][0] *= corr0; o[db][1] *= corr0; o[db][2] *= corr1; o[db][3] *= corr1; }
#pragma unroll
        for (int nb = 0; nb < KC / 8; nb++) {
            if (!(live & (1u << nb))) continue;
            const float p0 = exp2f(s[nb][0] - mu0), p1 = exp2f(s[nb][1] - mu0);
            const float p2 = exp2f(s[nb][2] - mu1), p3 = exp2f(s[nb][3] - mu1);
            l0 += p0 + p1; l1 += p2 + p3;
            // the C fragment of the scores is the A fragment of PV once key 2*tig sits in k-slot tig and key
            // 2*tig+1 in k-slot tig+4; V is read with the same permutation
            uint32_t ph[4], pl[4];
            tf32_split(p0, ph[0], pl[0]); tf32_split(p2, ph[1], pl[1]);
            tf32_split(p1, ph[2], pl[2]); tf32_split(p3, ph[3], pl[3]);
#pragma unroll
            for (int db = 0; db < KS; db++) {
                const float b0 = kv_f32(sV[nb * 8 + 2 * tig][db * 8 + g]), b1 = kv_f32(sV[nb * 8 + 2 * tig + 1][db * 8 + g]);
                if (SPLIT_KV) {
                    uint32_t h0, lo0, h1, lo1;
                    tf32_split(b0, h0, lo0); tf32_split(b1, h1, lo1);
                    mma_tf32(o[db], ph, h0, h1); mma_tf32(o[db], pl, h0, h1); mma_tf32(o[db], ph, lo0, lo1);
                } else {
                    mma_tf32(o[db], ph, __float_as_uint(b0), __float_as_uint(b1));
                }
            }
        }
    }
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1); l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1); l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
    if (act0) {
        const float inv = 1.0f / l0;
#pragma unroll
        for (int db = 0; db < KS; db++)
            *reinterpret_cast<float2 *>(O + (int64_t)r0 * D + hoff + db * 8 + 2 * tig) = make_float2(o[db][0] * inv, o[db][1] * inv);
        if (tig == 0) LSE[(int64_t)r0 * H + h] = (m0 + log2f(l0)) * LN2;
    }
    if (act1) {
        const float inv = 1.0f / l1;
#pragma unroll
        for (int db = 0; db < KS; db++)
            *reinterpret_cast<float2 *>(O + (int64_t)r1 * D + hoff + db * 8 + 2 * tig) = make_float2(o[db][2] * inv, o[db][3] * inv);
        if (tig == 0) LSE[(int64_t)r1 * H + h] = (m1 + log2f(l1)) * LN2;
    }
}

// --------------------------------------------------------------------------------------
// backward.  Per chunk of KC keys:
//   phase 1 (thread = query): w = exp(s - lse), ds = w (dO.v - delta) scale, dq += ds k; w and ds go
//                             to shared memory;
//   phase 2 (lane = key, warp = slice of head_dim): dK_key += sum_i ds[i] q_i, dV_key += sum_i w[i] dO_i
//                             over the tile's queries in index order.
// Rows of chain keys are written to the partial buffers (one row per (tile, chain slot)); rows of the
// tile's own keys go straight to dK/dV.  No atomics anywhere.
// --------------------------------------------------------------------------------------
template <int HD, int M>
struct BwdSmem {
    float sK[KC][HD + 4];
    float sV[KC][HD + 4];
    float sQ[M][HD];
    float sG[M][HD];
    float sW[M][KC + 1];
    float sS[M][KC + 1];
    int s_kid[KC], s_kend[KC];
};

template <int HD, int M, typename KVT>
__global__ void __launch_bounds__(M) attn_bwd_kernel(const float *__restrict__ Q, const KVT *__restrict__ K,
                                                     const KVT *__restrict__ V, const float *__restrict__ O,
                                                     const float *__restrict__ LSE, const float *__restrict__ dO,
                                                     float *__restrict__ dQ, float *__restrict__ dK,
                                                     float *__restrict__ dV, float *__restrict__ Pk,
                                                     float *__restrict__ Pv, const int32_t *__restrict__ sub_end,
                                                     const int64_t *__restrict__ chain_off,
                                                     const int32_t *__restrict__ chain_ids, int n, int H, float scale, int tile0,
                                                     BwdMask gmask) {
    extern __shared__ __align__(16) unsigned char smem_raw[];
    BwdSmem<HD, M> &S = *reinterpret_cast<BwdSmem<HD, M> *>(smem_raw);
    const int t = blockIdx.x + tile0, h = blockIdx.y, tid = threadIdx.x;
    const int D = H * HD, hoff = h * HD;
    const int i0 = t * M, i = i0 + tid;
    const bool active = i < n;
    const int nt = min(M, n - i0);
    const int64_t coff = chain_off[t];
    const int p = (int)(chain_off[t + 1] - coff);
    const int nkeys = p + nt;
    const int32_t *chain = chain_ids + coff;

    float q[HD], g[HD], dq[HD];
    float delta = 0.f;
#pragma unroll
    for (int c = 0; c < HD / 4; c++) {
        float4 x = make_float4(0.f, 0.f, 0.f, 0.f), y = x, o = x;
        if (active) {
            x = ld4(Q + (int64_t)i * D + hoff + c * 4);
            y = ld4(dO + (int64_t)i * D + hoff + c * 4);
            o = ld4(O + (int64_t)i * D + hoff + c * 4);
        }
        q[4 * c] = x.x; q[4 * c + 1] = x.y; q[4 * c + 2] = x.z; q[4 * c + 3] = x.w;
        g[4 * c] = y.x; g[4 * c + 1] = y.y; g[4 * c + 2] = y.z; g[4 * c + 3] = y.w;
        delta = fmaf(y.x, o.x, delta); delta = fmaf(y.y, o.y, delta);
        delta = fmaf(y.z, o.z, delta); delta = fmaf(y.w, o.w, delta);
        dq[4 * c] = dq[4 * c + 1] = dq[4 * c + 2] = dq[4 * c + 3] = 0.f;
        *reinterpret_cast<float4 *>(&S.sQ[tid][c * 4]) = x;
        *reinterpret_cast<float4 *>(&S.sG[tid][c * 4]) = y;
    }
    const float qs = scale * LOG2E;
    const float lse2 = active ? LSE[(int64_t)i * H + h] * LOG2E : 0.f;
    const int first_key = bwd_first_key(gmask, i, n);

    constexpr int NW = M / 32;          // warps = slices of head_dim in phase 2
    constexpr int SL = HD / NW;         // columns per slice
    const int lane = tid & 31, slice0 = (tid >> 5) * SL;

    for (int kc = 0; kc < nkeys; kc += KC) {
        const int cnt = min(KC, nkeys - kc);
        __syncthreads();
        stage_keys<HD, M, KVT>(K, V, sub_end, chain, p, i0, kc, cnt, D, hoff, S.s_kid, S.s_kend, S.sK, S.sV);
        // ---- phase 1 ----
        for (int j = 0; j < cnt; j++) {
            const bool vld = active && S.s_kid[j] <= i && i < S.s_kend[j];
            if (!__any_sync(0xffffffffu, vld)) {
                S.sW[tid][j] = 0.f; S.sS[tid][j] = 0.f;
                continue;
            }
            float d0 = 0.f, d1 = 0.f, e0 = 0.f, e1 = 0.f;
#pragma unroll
            for (int c = 0; c < HD / 4; c++) {
                float4 kk = *reinterpret_cast<const float4 *>(&S.sK[j][c * 4]);
                float4 vv = *reinterpret_cast<const float4 *>(&S.sV[j][c * 4]);
                d0 = fmaf(q[4 * c], kk.x, d0); d1 = fmaf(q[4 * c + 1], kk.y, d1);
                d0 = fmaf(q[4 * c + 2], kk.z, d0); d1 = fmaf(q[4 * c + 3], kk.w, d1);
                e0 = fmaf(g[4 * c], vv.x, e0); e1 = fmaf(g[4 * c + 1], vv.y, e1);
                e0 = fmaf(g[4 * c + 2], vv.z, e0); e1 = fmaf(g[4 * c + 3], vv.w, e1);
            }
            float w = vld ? exp2f((d0 + d1) * qs - lse2) : 0.f;
            float ds = w * ((e0 + e1) - delta) * scale;
            const bool keep = S.s_kid[j] >= first_key;             // dK/dV take this pair (dQ below always does)
            S.sW[tid][j] = keep ? w : 0.f; S.sS[tid][j] = keep ? ds : 0.f;
#pragma unroll
            for (int c = 0; c < HD / 4; c++) {
                float4 kk = *reinterpret_cast<const float4 *>(&S.sK[j][c * 4]);
                dq[4 * c] = fmaf(ds, kk.x, dq[4 * c]); dq[4 * c + 1] = fmaf(ds, kk.y, dq[4 * c + 1]);
                dq[4 * c + 2] = fmaf(ds, kk.z, dq[4 * c + 2]); dq[4 * c + 3] = fmaf(ds, kk.w, dq[4 * c + 3]);
            }
        }
        __syncthreads();
        // ---- phase 2 ----
        if (lane < cnt) {
            float ak[SL], av[SL];
#pragma unroll
            for (int c = 0; c < SL; c++) { ak[c] = 0.f; av[c] = 0.f; }
            const int kk_idx = kc + lane;
            // a tile key (index kk_idx - p inside the tile) is attended only by queries at or after it
            const int first_q = max(0, kc - p);
            for (int qi = first_q; qi < nt; qi++) {
                float w = S.sW[qi][lane], ds = S.sS[qi][lane];
                if (w == 0.f) continue;
#pragma unroll
                for (int c = 0; c < SL / 4; c++) {
                    float4 qq = *reinterpret_cast<const float4 *>(&S.sQ[qi][slice0 + c * 4]);
                    float4 gg = *reinterpret_cast<const float4 *>(&S.sG[qi][slice0 + c * 4]);
                    ak[4 * c] = fmaf(ds, qq.x, ak[4 * c]); ak[4 * c + 1] = fmaf(ds, qq.y, ak[4 * c + 1]);
                    ak[4 * c + 2] = fmaf(ds, qq.z, ak[4 * c + 2]); ak[4 * c + 3] = fmaf(ds, qq.w, ak[4 * c + 3]);
                    av[4 * c] = fmaf(w, gg.x, av[4 * c]); av[4 * c + 1] = fmaf(w, gg.y, av[4 * c + 1]);
                    av[4 * c + 2] = fmaf(w, gg.z, av[4 * c + 2]); av[4 * c + 3] = fmaf(w, gg.w, av[4 * c + 3]);
                }
            }
            float *ok, *ov;
            if (kk_idx < p) {
                ok = Pk + (coff + kk_idx) * D + hoff + slice0;
                ov = Pv + (coff + kk_idx) * D + hoff + slice0;
            } else {
                ok = dK + (int64_t)(i0 + kk_idx - p) * D + hoff + slice0;
                ov = dV + (int64_t)(i0 + kk_idx - p) * D + hoff + slice0;
            }
#pragma unroll
            for (int c = 0; c < SL / 4; c++) {
                *reinterpret_cast<float4 *>(ok + c * 4) = make_float4(ak[4 * c], ak[4 * c + 1], ak[4 * c + 2], ak[4 * c + 3]);
                *reinterpret_cast<float4 *>(ov + c * 4) = make_float4(av[4 * c], av[4 * c + 1], av[4 * c + 2], av[4 * c + 3]);
            }
        }
    }
    if (active) {
#pragma unroll
        for (int c = 0; c < HD / 4; c++)
            *reinterpret_cast<float4 *>(dQ + (int64_t)i * D + hoff + c * 4) =
                make_float4(dq[4 * c], dq[4 * c + 1], dq[4 * c + 2], dq[4 * c + 3]);
    }
}

// --------------------------------------------------------------------------------------
// backward on the tensor cores (same tiling and error compensation as attn_fwd_mma_kernel).
// Per chunk of 32 keys:
//   phase 1 (warp = 16 query rows): S = Q K^T, dP = dO V^T, P = exp2(S - lse), dS = P (dP - delta) scale,
//            dQ += dS K; P and dS go to shared memory;
//   phase 2 (warp = 16 keys x half of head_dim): dK = dS^T Q, dV = P^T dO, contracted over the tile's 64 queries
//            in index order.
// Output placement and the later reduction are those of attn_bwd_kernel.
// --------------------------------------------------------------------------------------
template <int HD, typename KVT>
struct BwdMmaSmem {
    typename SmemKV<KVT>::elem sKb[KC][HD + SmemKV<KVT>::PAD];     // one buffer: the next chunk is copied during phase 2
    typename SmemKV<KVT>::elem sVb[KC][HD + SmemKV<KVT>::PAD];
    float sQ[64][HD + 8];
    float sG[64][HD + 8];
    float sP[64][KC + 8];
    float sS[64][KC + 8];
    int s_kid[MAXKEYS], s_kend[MAXKEYS];
    unsigned s_live[4];
};

template <int HD, typename KVT>
__global__ void __launch_bounds__(128, HD <= 32 ? 4 : (sizeof(KVT) == 2 ? 3 : 1)) attn_bwd_mma_kernel(const float *__restrict__ Q, const KVT *__restrict__ K,
                                                           const KVT *__restrict__ V, const float *__restrict__ O,
                                                           const float *__restrict__ LSE, const float *__restrict__ dO,
                                                           float *__restrict__ dQ, float *__restrict__ dK,
                                                           float *__restrict__ dV, float *__restrict__ Pk,
                                                           float *__restrict__ Pv, const int32_t *__restrict__ sub_end,
                                                           const int64_t *__restrict__ chain_off,
                                                           const int32_t *__restrict__ chain_ids,
                                                           const int32_t *__restrict__ chain_end_all, int n, int H,
                                                           float scale, int tile0, BwdMask gmask) {
    constexpr int M = 64, KS = HD / 8;
    constexpr bool SPLIT_KV = sizeof(KVT) == 4;
    constexpr int NB2 = (KS + 1) / 2;          // head_dim blocks of 8 per warp in phase 2
    extern __shared__ __align__(16) unsigned char smem_raw[];
    BwdMmaSmem<HD, KVT> &S = *reinterpret_cast<BwdMmaSmem<HD, KVT> *>(smem_raw);
    typedef typename SmemKV<KVT>::elem SE;
    constexpr int SP = HD + SmemKV<KVT>::PAD;
    const int t = blockIdx.x + tile0, h = blockIdx.y, tid = threadIdx.x;
    const int warp = tid >> 5, lane = tid & 31, g = lane >> 2, tig = lane & 3;
    const int D = H * HD, hoff = h * HD;
    const int i0 = t * M;
    const int nt = min(M, n - i0);
    // tile-local query rows of this thread (pairing an early with a late group of 8 rows per warp, to even out the
    // triangular work between the warps, was measured slower: more 16 x 8 blocks become live)
    const int q0 = warp * 16 + g, q1 = q0 + 8;
    const int r0 = i0 + q0, r1 = i0 + q1;
    const bool act0 = r0 < n, act1 = r1 < n;
    const int64_t coff = chain_off[t];
    const int p = (int)(chain_off[t + 1] - coff);
    const int nkeys = p + nt;
    const int32_t *chain = chain_ids + coff;
    const float qs = scale * LOG2E;

    // Everything the prologue needs is requested at once: the tile's Q, dO and O rows by cp.async (O lands in the
    // area that later holds P; it is only needed for delta = dO.O), the key metadata by plain loads meanwhile.
    static_assert(64 * (HD + 8) <= 2 * 64 * (KC + 8), "the O rows are staged in the (contiguous) P and dS areas");
    float *sOflat = &S.sP[0][0];                 // viewed as [64][HD + 8]
    {
        constexpr int C4 = HD / 4;
        for (int idx = tid; idx < M * C4; idx += 128) {
            const int r = idx / C4, c = idx % C4;
            if (r < nt) {
                const int64_t off = (int64_t)(i0 + r) * D + hoff + c * 4;
                cp_async16(&S.sQ[r][c * 4], Q + off);
                cp_async16(&S.sG[r][c * 4], dO + off);
                cp_async16(sOflat + r * (HD + 8) + c * 4, O + off);
            } else {
                *reinterpret_cast<float4 *>(&S.sQ[r][c * 4]) = make_float4(0.f, 0.f, 0.f, 0.f);
                *reinterpret_cast<float4 *>(&S.sG[r][c * 4]) = make_float4(0.f, 0.f, 0.f, 0.f);
                *reinterpret_cast<float4 *>(sOflat + r * (HD + 8) + c * 4) = make_float4(0.f, 0.f, 0.f, 0.f);
            }
        }
        cp_async_commit();
    }
    load_key_meta(sub_end, chain, chain_end_all + coff, p, i0, nkeys, S.s_kid, S.s_kend);
    const float lse0 = act0 ? LSE[(int64_t)r0 * H + h] * LOG2E : 0.f;
    const float lse1 = act1 ? LSE[(int64_t)r1 * H + h] * LOG2E : 0.f;
    const int first0 = bwd_first_key(gmask, r0, n), first1 = bwd_first_key(gmask, r1, n);
    __syncthreads();                             // key metadata visible
    issue_chunk<HD, KVT>(K, V, S.s_kid, 0, min(KC, nkeys), D, hoff, S.sKb, S.sVb);
    asm volatile("cp.async.wait_group 1;" ::: "memory");      // the Q/dO/O group; chunk 0 may still be in flight
    __syncthreads();
    uint32_t qh[KS][4], ql[KS][4], gh[KS][4], gl[KS][4];
    float delta0 = 0.f, delta1 = 0.f;
#pragma unroll
    for (int ks = 0; ks < KS; ks++) {
        const int d0 = ks * 8 + tig;
        const float x0 = S.sQ[q0][d0], x1 = S.sQ[q1][d0], x2 = S.sQ[q0][d0 + 4], x3 = S.sQ[q1][d0 + 4];
        const float y0 = S.sG[q0][d0], y1 = S.sG[q1][d0], y2 = S.sG[q0][d0 + 4], y3 = S.sG[q1][d0 + 4];
        tf32_split(x0 * qs, qh[ks][0], ql[ks][0]); tf32_split(x1 * qs, qh[ks][1], ql[ks][1]);
        tf32_split(x2 * qs, qh[ks][2], ql[ks][2]); tf32_split(x3 * qs, qh[ks][3], ql[ks][3]);
        tf32_split(y0, gh[ks][0], gl[ks][0]); tf32_split(y1, gh[ks][1], gl[ks][1]);
        tf32_split(y2, gh[ks][2], gl[ks][2]); tf32_split(y3, gh[ks][3], gl[ks][3]);
        delta0 = fmaf(y0, sOflat[q0 * (HD + 8) + d0], delta0); delta0 = fmaf(y2, sOflat[q0 * (HD + 8) + d0 + 4], delta0);
        delta1 = fmaf(y1, sOflat[q1 * (HD + 8) + d0], delta1); delta1 = fmaf(y3, sOflat[q1 * (HD + 8) + d0 + 4], delta1);
    }
    delta0 += __shfl_xor_sync(0xffffffffu, delta0, 1); delta0 += __shfl_xor_sync(0xffffffffu, delta0, 2);
    delta1 += __shfl_xor_sync(0xffffffffu, delta1, 1); delta1 += __shfl_xor_sync(0xffffffffu, delta1, 2);
    float dq[KS][4];
#pragma unroll
    for (int db = 0; db < KS; db++) dq[db][0] = dq[db][1] = dq[db][2] = dq[db][3] = 0.f;

    const int mb = warp & 1;                    // phase 2: 16-key block of the chunk
    const int db0 = (warp >> 1) * NB2;          // phase 2: first head_dim block of this warp

    for (int kc = 0; kc < nkeys; kc += KC) {
        const int cnt = min(KC, nkeys - kc);
        SE (*sK)[SP] = S.sKb;
        SE (*sV)[SP] = S.sVb;
        cp_async_wait_all();
        __syncthreads();                              // chunk kc has landed; phase 2 of the previous chunk (and the
                                                      // delta pass over the O rows) is over
        // ---- phase 1 ----  (two key blocks at a time: four independent accumulator chains)
        unsigned live = 0;
#pragma unroll
        for (int nb2 = 0; nb2 < KC / 8; nb2 += 2) {
            bool vv[2][4];
            bool on[2];
            float c[2][4], e[2][4];
#pragma unroll
            for (int u = 0; u < 2; u++) {
                const int kA = (nb2 + u) * 8 + 2 * tig;
                const bool inA = kc + kA < nkeys, inB = kc + kA + 1 < nkeys;
                const int kidA = inA ? S.s_kid[kc + kA] : 0, kendA = inA ? S.s_kend[kc + kA] : 0;
                const int kidB = inB ? S.s_kid[kc + kA + 1] : 0, kendB = inB ? S.s_kend[kc + kA + 1] : 0;
                vv[u][0] = act0 && kidA <= r0 && r0 < kendA; vv[u][1] = act0 && kidB <= r0 && r0 < kendB;
                vv[u][2] = act1 && kidA <= r1 && r1 < kendA; vv[u][3] = act1 && kidB <= r1 && r1 < kendB;
                on[u] = __any_sync(0xffffffffu, vv[u][0] | vv[u][1] | vv[u][2] | vv[u][3]);
                if (on[u]) live |= 1u << (nb2 + u);
                c[u][0] = c[u][1] = c[u][2] = c[u][3] = 0.f;
                e[u][0] = e[u][1] = e[u][2] = e[u][3] = 0.f;
            }
            if (on[0] || on[1]) {
#pragma unroll
                for (int ks = 0; ks < KS; ks++) {
#pragma unroll
                    for (int u = 0; u < 2; u++) {
                        if (!on[u] && !ChunkBothHalves<HD>::value) continue;
                        const int nb = nb2 + u;
                        const float k0 = kv_f32(sK[nb * 8 + g][ks * 8 + tig]), k1 = kv_f32(sK[nb * 8 + g][ks * 8 + tig + 4]);
                        const float w0 = kv_f32(sV[nb * 8 + g][ks * 8 + tig]), w1 = kv_f32(sV[nb * 8 + g][ks * 8 + tig + 4]);
                        if (SPLIT_KV) {
                            uint32_t h0, lo0, h1, lo1, x0, y0, x1, y1;
                            tf32_split(k0, h0, lo0); tf32_split(k1, h1, lo1);
                            tf32_split(w0, x0, y0); tf32_split(w1, x1, y1);
                            mma_tf32(c[u], qh[ks], h0, h1); mma_tf32(e[u], gh[ks], x0, x1);
                            mma_tf32(c[u], ql[ks], h0, h1); mma_tf32(e[u], gl[ks], x0, x1);
                            mma_tf32(c[u], qh[ks], lo0, lo1); mma_tf32(e[u], gh[ks], y0, y1);
                        } else {
                            // bf16 store: single TF32 products throughout (see the forward kernel)
                            mma_tf32(c[u], qh[ks], __float_as_uint(k0), __float_as_uint(k1));
                            mma_tf32(e[u], gh[ks], __float_as_uint(w0), __float_as_uint(w1));
                        }
                    }
                }
            }
#pragma unroll
            for (int u = 0; u < 2; u++) {
                const int nb = nb2 + u, kA = nb * 8 + 2 * tig;
                float pw[4] = {0.f, 0.f, 0.f, 0.f}, ds[4] = {0.f, 0.f, 0.f, 0.f};
                if (on[u] || (ChunkBothHalves<HD>::value && (on[0] || on[1]))) {
                    pw[0] = vv[u][0] ? exp2f(c[u][0] - lse0) : 0.f; pw[1] = vv[u][1] ? exp2f(c[u][1] - lse0) : 0.f;
                    pw[2] = vv[u][2] ? exp2f(c[u][2] - lse1) : 0.f; pw[3] = vv[u][3] ? exp2f(c[u][3] - lse1) : 0.f;
                    ds[0] = pw[0] * (e[u][0] - delta0) * scale; ds[1] = pw[1] * (e[u][1] - delta0) * scale;
                    ds[2] = pw[2] * (e[u][2] - delta1) * scale; ds[3] = pw[3] * (e[u][3] - delta1) * scale;
                    // dQ += dS K  (C fragment reused as A fragment: key 2*tig in k-slot tig, key 2*tig+1 in k-slot tig+4)
                    uint32_t ah[4], al[4];
                    tf32_split(ds[0], ah[0], al[0]); tf32_split(ds[2], ah[1], al[1]);
                    tf32_split(ds[1], ah[2], al[2]); tf32_split(ds[3], ah[3], al[3]);
#pragma unroll
                    for (int db = 0; db < KS; db++) {
                        const float b0 = kv_f32(sK[nb * 8 + 2 * tig][db * 8 + g]), b1 = kv_f32(sK[nb * 8 + 2 * tig + 1][db * 8 + g]);
                        if (SPLIT_KV) {
                            uint32_t h0, lo0, h1, lo1;
                            tf32_split(b0, h0, lo0); tf32_split(b1, h1, lo1);
                            mma_tf32(dq[db], ah, h0, h1); mma_tf32(dq[db], al, h0, h1); mma_tf32(dq[db], ah, lo0, lo1);
                        } else {
                            mma_tf32(dq[db], ah, __float_as_uint(b0), __float_as_uint(b1));
                        }
                    }
                }
                if (gmask.mode != AGPT_GRAD_FULL && on[u]) {       // pairs that dK/dV do not take (dQ above took them all)
                    const int kidA = kc + kA < nkeys ? S.s_kid[kc + kA] : 0, kidB = kc + kA + 1 < nkeys ? S.s_kid[kc + kA + 1] : 0;
                    if (kidA < first0) { pw[0] = 0.f; ds[0] = 0.f; }
                    if (kidB < first0) { pw[1] = 0.f; ds[1] = 0.f; }
                    if (kidA < first1) { pw[2] = 0.f; ds[2] = 0.f; }
                    if (kidB < first1) { pw[3] = 0.f; ds[3] = 0.f; }
                }
                *reinterpret_cast<float2 *>(&S.sP[q0][kA]) = make_float2(pw[0], pw[1]);
                *reinterpret_cast<float2 *>(&S.sP[q1][kA]) = make_float2(pw[2], pw[3]);
                *reinterpret_cast<float2 *>(&S.sS[q0][kA]) = make_float2(ds[0], ds[1]);
                *reinterpret_cast<float2 *>(&S.sS[q1][kA]) = make_float2(ds[2], ds[3]);
            }
        }
        if (lane == 0) S.s_live[warp] = live;
        __syncthreads();
        // phase 2 does not touch K/V: the next chunk is copied while it runs
        if (kc + KC < nkeys) issue_chunk<HD, KVT>(K, V, S.s_kid, kc + KC, min(KC, nkeys - kc - KC), D, hoff, S.sKb, S.sVb);
        // ---- phase 2 ----
        if (mb * 16 < cnt) {
            float ak[NB2][4], av[NB2][4];
#pragma unroll
            for (int j = 0; j < NB2; j++) { ak[j][0] = ak[j][1] = ak[j][2] = ak[j][3] = 0.f; av[j][0] = av[j][1] = av[j][2] = av[j][3] = 0.f; }
            // a key of the tile itself is attended only by queries at or after it
            const int ks_first = max(0, kc + mb * 16 - p) / 8;
            for (int ks = ks_first; ks < M / 8; ks++) {
                if (!((S.s_live[ks >> 1] >> (2 * mb)) & 3u)) continue;       // the 16 queries x 16 keys are all masked
                const int qa = ks * 8 + tig, kA = mb * 16 + g;
                uint32_t sh[4], sl[4], ph[4], pl[4];
                tf32_split(S.sS[qa][kA], sh[0], sl[0]); tf32_split(S.sS[qa][kA + 8], sh[1], sl[1]);
                tf32_split(S.sS[qa + 4][kA], sh[2], sl[2]); tf32_split(S.sS[qa + 4][kA + 8], sh[3], sl[3]);
                tf32_split(S.sP[qa][kA], ph[0], pl[0]); tf32_split(S.sP[qa][kA + 8], ph[1], pl[1]);
                tf32_split(S.sP[qa + 4][kA], ph[2], pl[2]); tf32_split(S.sP[qa + 4][kA + 8], ph[3], pl[3]);
#pragma unroll
                for (int j = 0; j < NB2; j++) {
                    const int dcol = (db0 + j) * 8 + g;
                    if ((db0 + j) * 8 >= HD) continue;
                    uint32_t h0, lo0, h1, lo1;
                    tf32_split(S.sQ[qa][dcol], h0, lo0); tf32_split(S.sQ[qa + 4][dcol], h1, lo1);
                    mma_tf32(ak[j], sh, h0, h1);
                    if (SPLIT_KV) { mma_tf32(ak[j], sl, h0, h1); mma_tf32(ak[j], sh, lo0, lo1); }
                    tf32_split(S.sG[qa][dcol], h0, lo0); tf32_split(S.sG[qa + 4][dcol], h1, lo1);
                    mma_tf32(av[j], ph, h0, h1);
                    if (SPLIT_KV) { mma_tf32(av[j], pl, h0, h1); mma_tf32(av[j], ph, lo0, lo1); }
                }
            }
#pragma unroll
            for (int half = 0; half < 2; half++) {
                const int kl = mb * 16 + g + half * 8;       // key index inside the chunk
                if (kl >= cnt) continue;
                const int kk = kc + kl;
                float *ok, *ov;
                if (kk < p) { ok = Pk + (coff + kk) * D + hoff; ov = Pv + (coff + kk) * D + hoff; }
                else { ok = dK + (int64_t)(i0 + kk - p) * D + hoff; ov = dV + (int64_t)(i0 + kk - p) * D + hoff; }
#pragma unroll
                for (int j = 0; j < NB2; j++) {
                    if ((db0 + j) * 8 >= HD) continue;
                    const int dcol = (db0 + j) * 8 + 2 * tig;
                    *reinterpret_cast<float2 *>(ok + dcol) = make_float2(ak[j][2 * half], ak[j][2 * half + 1]);
                    *reinterpret_cast<float2 *>(ov + dcol) = make_float2(av[j][2 * half], av[j][2 * half + 1]);
                }
            }
        }
    }
    if (act0) {
#pragma unroll
        for (int db = 0; db < KS; db++)
            *reinterpret_cast<float2 *>(dQ + (int64_t)r0 * D + hoff + db * 8 + 2 * tig) = make_float2(dq[db][0], dq[db][1]);
    }
    if (act1) {
#pragma unroll
        for (int db = 0; db < KS; db++)
            *reinterpret_cast<float2 *>(dQ + (int64_t)r1 * D + hoff + db * 8 + 2 * tig) = make_float2(dq[db][2], dq[db][3]);
    }
}

// --------------------------------------------------------------------------------------
// backward, whole tile resident: attn_bwd_tile_kernel (head_dim 32 or 64, float32 store).
//
// Operands.  The tile's Q and dO rows and every key row the tile can attend (ancestor chain + the tile's own
// rows) are brought into shared memory ONCE (cp.async, raw float32) and converted in place to split half
// precision: x * s = hi + lo with hi, lo in fp16 and s a power of two chosen per (tile, head, tensor) so that the
// largest |x * s| lies in [1, 2).  hi carries 11 bits, lo the next 11 (its own rounding is 2^-24 absolute at this
// scale), so hi*hi + lo*hi + hi*lo reproduces the float32 product to about 2^-22 -- the accuracy of three TF32
// products -- while each mma.sync.m16n8k16 contracts twice as many elements as a TF32 m16n8k8, every fragment
// register carries two elements, and the operands take 4 bytes per element instead of 8.  The scales are exact
// (powers of two) and are divided out of the results.  A converted row is 4 * head_dim bytes: the hi halves then the lo
// halves, its 16-byte chunks XOR-swizzled with the row (chunk ^ row % 8), so that every fragment is one
// conflict-free ldmatrix.x4: "along the row" fragments plain, "across rows" fragments with .trans.
//
// Work.  After the staging barriers the warps never meet again.  A warp takes items from a shared counter and runs
// each from start to end with registers and read-only shared memory:
//   * row item (16 queries):  S = Q K^T and dP = dO V^T for the 16 rows against every block of 16 keys, P, dS,
//     dQ += dS K (the score fragments of two 8-key blocks are the A fragment of the next product); writes 16 dQ rows.
//   * key item (16 keys):     S^T = K Q^T and dP^T = V dO^T for the 16 keys against every block of 16 queries, P^T,
//     dS^T, dK += dS^T Q, dV += P^T dO;  writes 16 dK/dV rows (tile rows) or partial rows (chain keys).
// Scores are computed twice (once per orientation) instead of crossing shared memory between two phases: that
// costs two extra small products per block and removes every barrier, every P/dS store and reload from the loops.
// Each output element is produced by exactly one warp in a fixed order, so results do not depend on which warp
// took which item.
// --------------------------------------------------------------------------------------
__device__ __forceinline__ float ex2_ftz(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}
__device__ __forceinline__ uint32_t smem_u32_of(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void ldmatrix_x4(uint32_t (&r)[4], uint32_t smem_addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_addr));
}
__device__ __forceinline__ void ldmatrix_x4_trans(uint32_t (&r)[4], uint32_t smem_addr) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(smem_addr));
}
__device__ __forceinline__ void mma_f16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
// The two 8-key (or 8-query) halves of a 16 x 16 block are independent chains of products.  Where BOTH_HALVES is set the
// half none of whose pairs is valid is computed too (its results are masked to exact zeros), so that the two chains sit
// in one basic block and interleave; otherwise each half is skipped on its own.  Measured: head_dim 64 backward 35.9 ms
// against 37.6 ms on the 4M-node tree (eight warps per SM: the interleaving pays); head_dim 32 backward 51.7 against 49.6
// and forward 19.3 against 19.0 on the depth-32 trie (more spills, more warps to hide latency already).
#ifndef AGPT_TILE_BOTH_MIN_HD
#define AGPT_TILE_BOTH_MIN_HD 64
#endif
template <int HD> struct TileBothHalves { static constexpr bool bwd = HD >= AGPT_TILE_BOTH_MIN_HD, fwd = false; };
// (x, y) -> packed fp16 pair hi (x in the low half) and the packed pair lo of the remainders.  LO_UP: the remainders
// are stored times 2^11 (they are below 2^-11 |x|, so this keeps them in fp16's normal range and a small element keeps
// its full 22 bits next to a large one); products with such a lo are accumulated apart and enter times 2^-11.
#define LO_UP 2048.0f
#define LO_DOWN 0.00048828125f
template <bool UP>
__device__ __forceinline__ void f16_split2(float x, float y, uint32_t &hi, uint32_t &lo) {
    const __half2 h = __floats2half2_rn(x, y);
    const float2 f = __half22float2(h);
    const __half2 l = UP ? __floats2half2_rn((x - f.x) * LO_UP, (y - f.y) * LO_UP) : __floats2half2_rn(x - f.x, y - f.y);
    hi = *reinterpret_cast<const uint32_t *>(&h);
    lo = *reinterpret_cast<const uint32_t *>(&l);
}
__device__ __forceinline__ uint32_t f16_pack2(float x, float y) {
    const __half2 h = __floats2half2_rn(x, y);
    return *reinterpret_cast<const uint32_t *>(&h);
}
// A fragment of a product whose B operand is staged as (hi, lo * 2^11): P and dS enter times 2^11 (AUP), a = hi + lo
// as halves, and the factor of the B operand's lo part is a_s = hi * 2^-11, one half-precision multiply (that term is
// 2^-11 of the product, so the bits a_s loses below 2^-14 do not matter).  2^11 P <= 2048 and, with dO staged to a
// maximum in [0.25, 0.5), 2^11 |dS'| < 2^11 * 2 * 32 * 0.5 * 2 * 0.18 < 65504.
#define AUP 2048.0f
#define ADOWN 0.00048828125f
__device__ __forceinline__ uint32_t f16_down11(uint32_t h2) {
    const __half2 r = __hmul2(*reinterpret_cast<const __half2 *>(&h2), __float2half2_rn(LO_DOWN));
    return *reinterpret_cast<const uint32_t *>(&r);
}
// power of two s with max * s in [2^lift, 2^(lift+1)) (1 for max == 0), and its inverse
__device__ __forceinline__ void pow2_scale(uint32_t max_bits, int lift, float &s, float &inv) {
    int e = (int)(max_bits >> 23);
    e = e < 1 ? 127 + lift : (e > 250 ? 250 : e);
    s = __uint_as_float((uint32_t)(254 + lift - e) << 23);
    inv = __uint_as_float((uint32_t)(e - lift) << 23);
}

// One staged row holds head_dim floats raw, then head_dim hi halves followed by head_dim lo halves: 4 * head_dim bytes,
// head_dim / 4 chunks of 16 bytes, the low three bits of the chunk index XOR-ed with row % 8.

// Staging geometry of one thread: it owns chunk c of rows r0, r0 + s, r0 + 2 s, ... of every plane, s = threads /
// chunks per row.  s is a multiple of 8, so the swizzle term (row % 8) and with it the three byte offsets below are
// the same for all its rows up to a multiple of the row step: raw = where the raw float4 sits, hi / lo = where its
// four hi and four lo halves go after the conversion.
struct TileLane { int r0, c, raw, hi, lo; };
template <int HD>
__device__ __forceinline__ TileLane tile_lane(int tid) {
    constexpr int NCH = HD / 4;
    TileLane L;
    L.r0 = tid / NCH; L.c = tid % NCH;
    const int x = L.r0 & 7, row = L.r0 * (HD * 4), half = (L.c & 1) << 3;
    L.raw = row + ((L.c ^ x) << 4);
    L.hi = row + (((L.c >> 1) ^ x) << 4) + half;
    L.lo = row + (((HD / 8 + (L.c >> 1)) ^ x) << 4) + half;
    return L;
}
__device__ __forceinline__ float abs_max4(float m, float4 a) {
    return fmaxf(m, fmaxf(fmaxf(fabsf(a.x), fabsf(a.y)), fmaxf(fabsf(a.z), fabsf(a.w))));
}
// In-place conversion of the thread's chunk (row offset o) of two planes: the eight lanes that own the chunks of one
// row read them, the warp synchronises, and each lane writes its four hi and four lo halves into the row's hi and lo
// part.  Called by whole warps.
__device__ __forceinline__ void tile_convert2(unsigned char *pa, unsigned char *pb, const TileLane &L, int o, float sa, float sb) {
    const float4 a = *reinterpret_cast<const float4 *>(pa + L.raw + o), b = *reinterpret_cast<const float4 *>(pb + L.raw + o);
    uint2 ah, al, bh, bl;
    f16_split2<true>(a.x * sa, a.y * sa, ah.x, al.x); f16_split2<true>(a.z * sa, a.w * sa, ah.y, al.y);
    f16_split2<true>(b.x * sb, b.y * sb, bh.x, bl.x); f16_split2<true>(b.z * sb, b.w * sb, bh.y, bl.y);
    __syncwarp();
    *reinterpret_cast<uint2 *>(pa + L.hi + o) = ah; *reinterpret_cast<uint2 *>(pa + L.lo + o) = al;
    *reinterpret_cast<uint2 *>(pb + L.hi + o) = bh; *reinterpret_cast<uint2 *>(pb + L.lo + o) = bl;
    __syncwarp();
}

// bfloat16 store: a key row arrives as head_dim bf16 (head_dim / 8 chunks of 16 bytes).  The raw chunk c is parked in the
// row's lo part (chunk head_dim / 8 + c, swizzled like every chunk) and converted to the hi chunk c of the same row: a
// bf16 value has 8 significant bits, so its scaled fp16 image is exact and the row has no lo part.  With such a store
// every product is a single fp16 product (Q, dO, P and dS are rounded to their 11-bit hi halves): about 1e-3 relative,
// below the store's own rounding (2^-9).  The thread that copied a chunk is the one that converts it.
struct KvLane { int r0, raw, hi; };
template <int HD>
__device__ __forceinline__ KvLane kv_lane(int tid) {
    constexpr int NCHK = HD / 8;
    KvLane L;
    L.r0 = tid / NCHK;
    const int c = tid % NCHK, x = L.r0 & 7, row = L.r0 * (HD * 4);
    L.raw = row + (((NCHK + c) ^ x) << 4);
    L.hi = row + ((c ^ x) << 4);
    return L;
}
__device__ __forceinline__ float abs_max_bf16x8(float m, uint4 a) {
    const uint32_t w[4] = {a.x, a.y, a.z, a.w};
#pragma unroll
    for (int j = 0; j < 4; j++)
        m = fmaxf(m, fmaxf(fabsf(__uint_as_float(w[j] << 16)), fabsf(__uint_as_float(w[j] & 0xffff0000u))));
    return m;
}
__device__ __forceinline__ void kv_convert_bf16(unsigned char *pa, const KvLane &L, int o, float sa) {
    const uint4 a = *reinterpret_cast<const uint4 *>(pa + L.raw + o);
    const uint32_t w[4] = {a.x, a.y, a.z, a.w};
    uint32_t h[4];
#pragma unroll
    for (int j = 0; j < 4; j++) h[j] = f16_pack2(__uint_as_float(w[j] << 16) * sa, __uint_as_float(w[j] & 0xffff0000u) * sa);
    *reinterpret_cast<uint4 *>(pa + L.hi + o) = make_uint4(h[0], h[1], h[2], h[3]);
}

constexpr size_t bwd_tile_smem_bytes(int hd, int maxk) {
    return (size_t)(2 * 64 + 2 * maxk) * (size_t)(hd * 4) + (size_t)maxk * 8 + 3 * 64 * 4 + 32;
}

template <int HD, int NW, int MINB, typename KVT>
__global__ void __launch_bounds__(NW * 32, MINB)
attn_bwd_tile_kernel(const float *__restrict__ Q, const KVT *__restrict__ K, const KVT *__restrict__ V,
                     const float *__restrict__ O, const float *__restrict__ LSE, const float *__restrict__ dO,
                     float *__restrict__ dQ, float *__restrict__ dK, float *__restrict__ dV, float *__restrict__ Pk,
                     float *__restrict__ Pv, const int32_t *__restrict__ sub_end, const int64_t *__restrict__ chain_off,
                     const int32_t *__restrict__ chain_ids, const int32_t *__restrict__ chain_end_all, int n, int H,
                     float scale, int tile0, int maxk, int dbg, BwdMask gmask) {
    constexpr int M = 64, NT = NW * 32, TILE_ROW_BYTES = HD * 4, KS = HD / 16, NDB = HD / 8, NCH = HD / 4;
    constexpr bool LP = sizeof(KVT) == 2;              // bfloat16 store: single fp16 products, no lo parts
    extern __shared__ __align__(128) unsigned char tile_smem_raw[];
    unsigned char *sQ = tile_smem_raw, *sG = sQ + M * TILE_ROW_BYTES, *sK = sG + M * TILE_ROW_BYTES;
    unsigned char *sV = sK + (size_t)maxk * TILE_ROW_BYTES;
    int2 *s_meta = reinterpret_cast<int2 *>(sV + (size_t)maxk * TILE_ROW_BYTES);   // [maxk] {key id, key subtree end}
    float *sLse = reinterpret_cast<float *>(s_meta + maxk);                          // [64]  lse * log2(e)
    float *sDelta = sLse + M;                                                        // [64]  dO . O
    int *sFirst = reinterpret_cast<int *>(sDelta + M);                               // [64]  first key id each query feeds in dK/dV
    uint32_t *s_max = reinterpret_cast<uint32_t *>(sFirst + M);                      // [4]   max |x| of Q, K, V, dO (float bits)
    int *s_ctr = reinterpret_cast<int *>(s_max + 4);

    const int t = blockIdx.x + tile0, h = blockIdx.y, tid = threadIdx.x;
    const int lane = tid & 31, g = lane >> 2, tig = lane & 3;
    const int D = H * HD, hoff = h * HD;
    const int i0 = t * M;
    const int nt = min(M, n - i0);
    const int64_t coff = chain_off[t];
    const int p = (int)(chain_off[t + 1] - coff);
    const int nkeys = p + nt;
    const int nkp = (nkeys + 15) & ~15;                // rows staged (zero rows beyond nkeys)
    const int32_t *chain = chain_ids + coff;
    const int32_t *chain_end = chain_end_all + coff;

    // ---- stage 1: raw rows by cp.async (chunk c of row r goes to chunk c ^ r % 8), O rows to registers ----
    if (tid < 4) s_max[tid] = 0u;
    if (tid == 0) *s_ctr = 0;
    constexpr int RSTEP = NT / NCH, OSTEP = RSTEP * TILE_ROW_BYTES;
    static_assert(NT % NCH == 0 && RSTEP % 8 == 0, "a thread's rows must share their swizzle term");
    constexpr int UQ = (M + RSTEP - 1) / RSTEP;
    const TileLane L = tile_lane<HD>(tid);
    float4 ox[UQ];
#pragma unroll
    for (int u = 0; u < UQ; u++) {
        const int r = L.r0 + u * RSTEP, o = L.raw + u * OSTEP;
        ox[u] = make_float4(0.f, 0.f, 0.f, 0.f);
        if (r < M) {
            if (r < nt) {
                const int64_t off = (int64_t)(i0 + r) * D + hoff + L.c * 4;
                cp_async16(sQ + o, Q + off); cp_async16(sG + o, dO + off);
                ox[u] = ld4(O + off);
            } else {
                *reinterpret_cast<float4 *>(sQ + o) = make_float4(0.f, 0.f, 0.f, 0.f);
                *reinterpret_cast<float4 *>(sG + o) = make_float4(0.f, 0.f, 0.f, 0.f);
            }
        }
    }
    constexpr int RSTEPK = NT / (HD / 8), OSTEPK = RSTEPK * TILE_ROW_BYTES;
    static_assert(NT % (HD / 8) == 0 && RSTEPK % 8 == 0, "a thread's key rows must share their swizzle term");
    const KvLane LK = kv_lane<HD>(tid);
    if constexpr (LP) {
        for (int r = LK.r0, o = LK.raw; r < nkp; r += RSTEPK, o += OSTEPK) {
            if (r < nkeys) {
                const int kid = r < p ? __ldg(chain + r) : i0 + (r - p);
                const int64_t off = (int64_t)kid * D + hoff + (tid % (HD / 8)) * 8;
                cp_async16(sK + o, K + off); cp_async16(sV + o, V + off);
            } else {
                *reinterpret_cast<uint4 *>(sK + o) = make_uint4(0u, 0u, 0u, 0u);
                *reinterpret_cast<uint4 *>(sV + o) = make_uint4(0u, 0u, 0u, 0u);
            }
        }
    } else {
        for (int r = L.r0, o = L.raw; r < nkp; r += RSTEP, o += OSTEP) {
            if (r < nkeys) {
                const int kid = r < p ? __ldg(chain + r) : i0 + (r - p);
                const int64_t off = (int64_t)kid * D + hoff + L.c * 4;
                cp_async16(sK + o, K + off); cp_async16(sV + o, V + off);
            } else {
                *reinterpret_cast<float4 *>(sK + o) = make_float4(0.f, 0.f, 0.f, 0.f);
                *reinterpret_cast<float4 *>(sV + o) = make_float4(0.f, 0.f, 0.f, 0.f);
            }
        }
    }
    cp_async_commit();
    for (int j = tid; j < nkp; j += NT) {
        int kid = 0x7fffffff, kend = 0;
        if (j < p) { kid = __ldg(chain + j); kend = __ldg(chain_end + j); }
        else if (j < nkeys) { kid = i0 + (j - p); kend = __ldg(sub_end + kid); }
        s_meta[j] = make_int2(kid, kend);
    }
    if (tid < M) {
        sLse[tid] = tid < nt ? __ldg(LSE + (int64_t)(i0 + tid) * H + h) * LOG2E : 0.f;
        sFirst[tid] = bwd_first_key(gmask, i0 + tid, n);
    }
    cp_async_wait_all();                 // this thread's own chunks have landed (pass A reads only those)

    // ---- stage 2 (pass A): maxima of |x| per tensor, delta = dO . O per row ----
    {
        float mq = 0.f, mg = 0.f, mk = 0.f, mv = 0.f;
#pragma unroll
        for (int u = 0; u < UQ; u++) {       // whole warps enter or skip an iteration (a warp holds four whole rows)
            const int r = L.r0 + u * RSTEP, o = L.raw + u * OSTEP;
            if (r < M) {
                const float4 a = *reinterpret_cast<const float4 *>(sQ + o), b = *reinterpret_cast<const float4 *>(sG + o);
                mq = abs_max4(mq, a); mg = abs_max4(mg, b);
                float d = b.x * ox[u].x;
                d = fmaf(b.y, ox[u].y, d); d = fmaf(b.z, ox[u].z, d); d = fmaf(b.w, ox[u].w, d);
#pragma unroll
                for (int o = 1; o < NCH; o <<= 1) d += __shfl_xor_sync(0xffffffffu, d, o);
                if (L.c == 0) sDelta[r] = d;
            }
        }
        if constexpr (LP) {
            for (int r = LK.r0, o = LK.raw; r < nkp; r += RSTEPK, o += OSTEPK) {
                mk = abs_max_bf16x8(mk, *reinterpret_cast<const uint4 *>(sK + o));
                mv = abs_max_bf16x8(mv, *reinterpret_cast<const uint4 *>(sV + o));
            }
        } else {
            for (int r = L.r0, o = L.raw; r < nkp; r += RSTEP, o += OSTEP) {
                mk = abs_max4(mk, *reinterpret_cast<const float4 *>(sK + o));
                mv = abs_max4(mv, *reinterpret_cast<const float4 *>(sV + o));
            }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            mq = fmaxf(mq, __shfl_xor_sync(0xffffffffu, mq, o)); mg = fmaxf(mg, __shfl_xor_sync(0xffffffffu, mg, o));
            mk = fmaxf(mk, __shfl_xor_sync(0xffffffffu, mk, o)); mv = fmaxf(mv, __shfl_xor_sync(0xffffffffu, mv, o));
        }
        if (lane == 0) {                     // non-negative floats order like their bit patterns
            atomicMax(&s_max[0], __float_as_uint(mq)); atomicMax(&s_max[1], __float_as_uint(mk));
            atomicMax(&s_max[2], __float_as_uint(mv)); atomicMax(&s_max[3], __float_as_uint(mg));
        }
    }
    __syncthreads();
    float sclQ, invQ, sclK, invK, sclV, invV, sclG, invG;
    pow2_scale(s_max[0], 0, sclQ, invQ); pow2_scale(s_max[1], 0, sclK, invK);
    pow2_scale(s_max[2], 0, sclV, invV); pow2_scale(s_max[3], -2, sclG, invG);

    // ---- stage 3 (pass B): convert in place ----
#pragma unroll
    for (int u = 0; u < UQ; u++)
        if (L.r0 + u * RSTEP < M) tile_convert2(sQ, sG, L, u * OSTEP, sclQ, sclG);
    if constexpr (LP) {
        for (int r = LK.r0, o = 0; r < nkp; r += RSTEPK, o += OSTEPK) { kv_convert_bf16(sK, LK, o, sclK); kv_convert_bf16(sV, LK, o, sclV); }
    } else {
        for (int r = L.r0, o = 0; r < nkp; r += RSTEP, o += OSTEP) tile_convert2(sK, sV, L, o, sclK, sclV);
    }
    __syncthreads();

    // units: S' = (Q sQ)(K sK)^T, dP' = (dO sG)(V sV)^T, P' = 2^11 P, dS' = P' (dP' - delta sG sV) scale = 2^11 dS sG sV
    const float fS = scale * LOG2E * invQ * invK;       // log2-domain score = S' * fS
    // dQ = (dS' K') / (2^11 sG sV sK), dK = (dS'^T Q') / (2^11 sG sV sQ), dV = (P'^T dO') / (2^11 sG); delta enters dS' as delta sG sV.
    // The powers of two are applied one after the other, never as one product that could leave the float range.

    // ldmatrix lane addressing: lane l names row l % 8 of matrix l / 8 (rows of 16 bytes).
    const int l8 = lane & 7, mi = lane >> 3;
    // B fragments of an 8-row block for k-step ks (16 dims): matrices {hi chunk 2ks, hi 2ks+1, lo 2ks, lo 2ks+1}
    const uint32_t bRow = (uint32_t)(l8 * TILE_ROW_BYTES);
    const int bC = (mi & 1) + (mi >> 1) * NDB;          // + 2 ks
    // A fragments of a 16-row block for k-step ks: matrices {rows 0-7 chunk 2ks, rows 8-15 chunk 2ks, rows 0-7 chunk 2ks+1,
    // rows 8-15 chunk 2ks+1} (+4 for the lo part); the .trans fragments of a 16-row block for dims 8 db..: {hi rows 0-7,
    // hi rows 8-15, lo rows 0-7, lo rows 8-15} of chunk db (+4 for lo)
    const uint32_t aRow = (uint32_t)((l8 + (mi & 1) * 8) * TILE_ROW_BYTES);
    const int aC = mi >> 1;                             // + 2 ks (+ 4 for lo)
    const int tC = (mi >> 1) * NDB;                     // + db
    const uint32_t uQ = smem_u32_of(sQ), uG = smem_u32_of(sG), uK = smem_u32_of(sK), uV = smem_u32_of(sV);

    const int nkb = nkp >> 4;                    // key items
    const int npc = (p + 15) >> 4;               // key items that hold chain keys (the heaviest: attended by most rows)
    const int n_items = nkb + 4;

    for (;;) {
        int it = 0;
        if (lane == 0) it = atomicAdd(s_ctr, 1);
        it = __shfl_sync(0xffffffffu, it, 0);
        if (it >= n_items) break;
        // order: chain key items, row items (last rows first), the tile's own key items
        int kind, which;
        if (it < npc) { kind = 1; which = it; }
        else if (it < npc + 4) { kind = 0; which = 3 - (it - npc); }
        else { kind = 1; which = it - 4; }
        if ((dbg >> kind) & 1) continue;

        if (kind == 0) {
            // ================= row item: 16 queries, every block of 16 keys =================
            const int rg = which;
            if (rg * 16 >= nt) continue;                                   // rows beyond the end of the plan
            const int q0 = rg * 16 + g, q1 = q0 + 8;
            const int r0 = i0 + q0, r1 = i0 + q1;
            uint32_t qh[KS][4], ql[KS][4], gh[KS][4], gl[KS][4];
#pragma unroll
            for (int ks = 0; ks < KS; ks++) {
                const uint32_t o = (uint32_t)(rg * 16 * TILE_ROW_BYTES) + aRow;
                const uint32_t ch = (uint32_t)(((2 * ks + aC) ^ l8) << 4), cl = (uint32_t)(((2 * ks + aC + NDB) ^ l8) << 4);
                ldmatrix_x4(qh[ks], uQ + o + ch); ldmatrix_x4(gh[ks], uG + o + ch);
                if constexpr (!LP) { ldmatrix_x4(ql[ks], uQ + o + cl); ldmatrix_x4(gl[ks], uG + o + cl); }
            }
            const float lse0 = sLse[q0], lse1 = sLse[q1], dl0 = sDelta[q0] * sclG * sclV, dl1 = sDelta[q1] * sclG * sclV;
            float dq[NDB][4];
#pragma unroll
            for (int db = 0; db < NDB; db++) dq[db][0] = dq[db][1] = dq[db][2] = dq[db][3] = 0.f;
            // the rows of this group attend the chain and the tile's keys up to their own position
            const int kp_lim = min((nkeys + 15) >> 4, (p + rg * 16 + 16 + 15) >> 4);
            for (int kp = 0; kp < kp_lim; kp++) {
                bool vld[2][4];
                bool on[2];
#pragma unroll
                for (int u = 0; u < 2; u++) {
                    const int4 mk = *reinterpret_cast<const int4 *>(&s_meta[kp * 16 + u * 8 + 2 * tig]);   // keys 2*tig, 2*tig+1 of the block
                    vld[u][0] = mk.x <= r0 && r0 < mk.y; vld[u][1] = mk.z <= r0 && r0 < mk.w;
                    vld[u][2] = mk.x <= r1 && r1 < mk.y; vld[u][3] = mk.z <= r1 && r1 < mk.w;
                    on[u] = __any_sync(0xffffffffu, vld[u][0] | vld[u][1] | vld[u][2] | vld[u][3]);
                }
                if (!(on[0] || on[1])) continue;
                float ds[2][4];
#pragma unroll
                for (int u = 0; u < 2; u++) {
                    ds[u][0] = ds[u][1] = ds[u][2] = ds[u][3] = 0.f;
                    if (!on[u] && !TileBothHalves<HD>::bwd) continue;                  // warp-uniform
                    float c[4] = {0.f, 0.f, 0.f, 0.f}, cx[4] = {0.f, 0.f, 0.f, 0.f};
                    float e[4] = {0.f, 0.f, 0.f, 0.f}, ex[4] = {0.f, 0.f, 0.f, 0.f};
                    const uint32_t rowb = (uint32_t)((kp * 16 + u * 8) * TILE_ROW_BYTES) + bRow;
#pragma unroll
                    for (int ks = 0; ks < KS; ks++) {
                        const uint32_t o = rowb + (uint32_t)(((2 * ks + bC) ^ l8) << 4);
                        uint32_t kf[4], vf[4];                 // {b0 hi, b1 hi, b0 lo, b1 lo}
                        ldmatrix_x4(kf, uK + o); ldmatrix_x4(vf, uV + o);
                        mma_f16(c, qh[ks], kf[0], kf[1]); mma_f16(e, gh[ks], vf[0], vf[1]);
                        if constexpr (!LP) {
                            mma_f16(cx, ql[ks], kf[0], kf[1]); mma_f16(ex, gl[ks], vf[0], vf[1]);
                            mma_f16(cx, qh[ks], kf[2], kf[3]); mma_f16(ex, gh[ks], vf[2], vf[3]);
                        }
                    }
#pragma unroll
                    for (int j = 0; j < 4; j++) {
                        const float sc = fmaf(cx[j], LO_DOWN, c[j]), dp = fmaf(ex[j], LO_DOWN, e[j]);
                        const float pw = vld[u][j] ? ex2_ftz(fmaf(sc, fS, j < 2 ? -lse0 : -lse1)) : 0.f;
                        ds[u][j] = pw * (dp - (j < 2 ? dl0 : dl1)) * (scale * AUP);
                    }
                }
                // dQ += dS K over the 16 keys: the score fragments of the two 8-key blocks are the A fragment
                uint32_t ah[4], al[4], as[4];
                f16_split2<false>(ds[0][0], ds[0][1], ah[0], al[0]); f16_split2<false>(ds[0][2], ds[0][3], ah[1], al[1]);
                f16_split2<false>(ds[1][0], ds[1][1], ah[2], al[2]); f16_split2<false>(ds[1][2], ds[1][3], ah[3], al[3]);
#pragma unroll
                for (int j = 0; j < 4; j++) as[j] = f16_down11(ah[j]);
                const uint32_t rowt = uK + (uint32_t)(kp * 16 * TILE_ROW_BYTES) + aRow;
#pragma unroll
                for (int db = 0; db < NDB; db++) {
                    uint32_t kt[4];                            // {b0 hi, b1 hi, b0 lo, b1 lo}: keys 0-7 / 8-15 of the block, dims 8 db..
                    ldmatrix_x4_trans(kt, rowt + (uint32_t)(((db + tC) ^ l8) << 4));
                    mma_f16(dq[db], ah, kt[0], kt[1]);
                    if constexpr (!LP) { mma_f16(dq[db], al, kt[0], kt[1]); mma_f16(dq[db], as, kt[2], kt[3]); }
                }
            }
            if (r0 < n) {
#pragma unroll
                for (int db = 0; db < NDB; db++)
                    *reinterpret_cast<float2 *>(dQ + (int64_t)r0 * D + hoff + db * 8 + 2 * tig) = make_float2(dq[db][0] * ADOWN * invG * invV * invK, dq[db][1] * ADOWN * invG * invV * invK);
            }
            if (r1 < n) {
#pragma unroll
                for (int db = 0; db < NDB; db++)
                    *reinterpret_cast<float2 *>(dQ + (int64_t)r1 * D + hoff + db * 8 + 2 * tig) = make_float2(dq[db][2] * ADOWN * invG * invV * invK, dq[db][3] * ADOWN * invG * invV * invK);
            }
        } else {
            // ================= key item: 16 keys, every block of 16 queries =================
            const int kb = which;
            const int kA = kb * 16 + g, kB = kA + 8;
            const int2 mA = s_meta[kA], mB = s_meta[kB];
            uint32_t kh[KS][4], kl[KS][4], vh[KS][4], vl[KS][4];
#pragma unroll
            for (int ks = 0; ks < KS; ks++) {
                const uint32_t o = (uint32_t)(kb * 16 * TILE_ROW_BYTES) + aRow;
                const uint32_t ch = (uint32_t)(((2 * ks + aC) ^ l8) << 4), cl = (uint32_t)(((2 * ks + aC + NDB) ^ l8) << 4);
                ldmatrix_x4(kh[ks], uK + o + ch); ldmatrix_x4(vh[ks], uV + o + ch);
                if constexpr (!LP) { ldmatrix_x4(kl[ks], uK + o + cl); ldmatrix_x4(vl[ks], uV + o + cl); }
            }
            float dk[NDB][4], dv[NDB][4];
#pragma unroll
            for (int db = 0; db < NDB; db++) {
                dk[db][0] = dk[db][1] = dk[db][2] = dk[db][3] = 0.f;
                dv[db][0] = dv[db][1] = dv[db][2] = dv[db][3] = 0.f;
            }
            // a key of the tile itself is attended only by queries at or after it
            const int qp_first = max(0, kb * 16 - p) >> 4;
            const int qp_end = (nt + 15) >> 4;
            for (int qp = qp_first; qp < qp_end; qp++) {
                bool vld[2][4];
                bool on[2];
#pragma unroll
                for (int u = 0; u < 2; u++) {
                    const int rq0 = i0 + qp * 16 + u * 8 + 2 * tig, rq1 = rq0 + 1;
                    const int2 fk = *reinterpret_cast<const int2 *>(&sFirst[qp * 16 + u * 8 + 2 * tig]);
                    vld[u][0] = mA.x <= rq0 && rq0 < mA.y && mA.x >= fk.x; vld[u][1] = mA.x <= rq1 && rq1 < mA.y && mA.x >= fk.y;
                    vld[u][2] = mB.x <= rq0 && rq0 < mB.y && mB.x >= fk.x; vld[u][3] = mB.x <= rq1 && rq1 < mB.y && mB.x >= fk.y;
                    on[u] = __any_sync(0xffffffffu, vld[u][0] | vld[u][1] | vld[u][2] | vld[u][3]);
                }
                if (!(on[0] || on[1])) continue;
                float ds[2][4], pw[2][4];
#pragma unroll
                for (int u = 0; u < 2; u++) {
                    ds[u][0] = ds[u][1] = ds[u][2] = ds[u][3] = 0.f;
                    pw[u][0] = pw[u][1] = pw[u][2] = pw[u][3] = 0.f;
                    if (!on[u] && !TileBothHalves<HD>::bwd) continue;                  // warp-uniform
                    float c[4] = {0.f, 0.f, 0.f, 0.f}, cx[4] = {0.f, 0.f, 0.f, 0.f};
                    float e[4] = {0.f, 0.f, 0.f, 0.f}, ex[4] = {0.f, 0.f, 0.f, 0.f};
                    const int qr = qp * 16 + u * 8;
                    const uint32_t rowb = (uint32_t)(qr * TILE_ROW_BYTES) + bRow;
#pragma unroll
                    for (int ks = 0; ks < KS; ks++) {
                        const uint32_t o = rowb + (uint32_t)(((2 * ks + bC) ^ l8) << 4);
                        uint32_t qf[4], gf[4];                 // {b0 hi, b1 hi, b0 lo, b1 lo}
                        ldmatrix_x4(qf, uQ + o); ldmatrix_x4(gf, uG + o);
                        mma_f16(c, kh[ks], qf[0], qf[1]); mma_f16(e, vh[ks], gf[0], gf[1]);
                        if constexpr (!LP) {
                            mma_f16(cx, kl[ks], qf[0], qf[1]); mma_f16(ex, vl[ks], gf[0], gf[1]);
                            mma_f16(cx, kh[ks], qf[2], qf[3]); mma_f16(ex, vh[ks], gf[2], gf[3]);
                        }
                    }
                    const float2 ls = *reinterpret_cast<const float2 *>(&sLse[qr + 2 * tig]);
                    const float2 dl = *reinterpret_cast<const float2 *>(&sDelta[qr + 2 * tig]);
#pragma unroll
                    for (int j = 0; j < 4; j++) {
                        const float sc = fmaf(cx[j], LO_DOWN, c[j]), dp = fmaf(ex[j], LO_DOWN, e[j]);
                        const float pr = vld[u][j] ? ex2_ftz(fmaf(sc, fS, (j & 1) ? -ls.y : -ls.x)) : 0.f;
                        pw[u][j] = pr * AUP;
                        ds[u][j] = pw[u][j] * (dp - ((j & 1) ? dl.y : dl.x) * sclG * sclV) * scale;
                    }
                }
                // dK += dS^T Q, dV += P^T dO over the 16 queries
                uint32_t sh[4], sl[4], ss[4], ph[4], pl[4], ps[4];
#pragma unroll
                for (int u = 0; u < 2; u++) {
                    f16_split2<false>(ds[u][0], ds[u][1], sh[2 * u], sl[2 * u]); f16_split2<false>(ds[u][2], ds[u][3], sh[2 * u + 1], sl[2 * u + 1]);
                    f16_split2<false>(pw[u][0], pw[u][1], ph[2 * u], pl[2 * u]); f16_split2<false>(pw[u][2], pw[u][3], ph[2 * u + 1], pl[2 * u + 1]);
                    ss[2 * u] = f16_down11(sh[2 * u]); ss[2 * u + 1] = f16_down11(sh[2 * u + 1]);
                    ps[2 * u] = f16_down11(ph[2 * u]); ps[2 * u + 1] = f16_down11(ph[2 * u + 1]);
                }
                const uint32_t ro = (uint32_t)(qp * 16 * TILE_ROW_BYTES) + aRow;
#pragma unroll
                for (int db = 0; db < NDB; db++) {
                    uint32_t qt[4], gt[4];                     // {b0 hi, b1 hi, b0 lo, b1 lo}: queries 0-7 / 8-15 of the block, dims 8 db..
                    const uint32_t co = (uint32_t)(((db + tC) ^ l8) << 4);
                    ldmatrix_x4_trans(qt, uQ + ro + co); ldmatrix_x4_trans(gt, uG + ro + co);
                    mma_f16(dk[db], sh, qt[0], qt[1]); mma_f16(dv[db], ph, gt[0], gt[1]);
                    if constexpr (!LP) {
                        mma_f16(dk[db], sl, qt[0], qt[1]); mma_f16(dv[db], pl, gt[0], gt[1]);
                        mma_f16(dk[db], ss, qt[2], qt[3]); mma_f16(dv[db], ps, gt[2], gt[3]);
                    }
                }
            }
#pragma unroll
            for (int half = 0; half < 2; half++) {
                const int kk = kb * 16 + g + half * 8;
                if (kk >= nkeys) continue;
                float *ok, *ov;
                if (kk < p) { ok = Pk + (coff + kk) * D + hoff; ov = Pv + (coff + kk) * D + hoff; }
                else { ok = dK + (int64_t)(i0 + kk - p) * D + hoff; ov = dV + (int64_t)(i0 + kk - p) * D + hoff; }
#pragma unroll
                for (int db = 0; db < NDB; db++) {
                    *reinterpret_cast<float2 *>(ok + db * 8 + 2 * tig) = make_float2(dk[db][2 * half] * ADOWN * invG * invV * invQ, dk[db][2 * half + 1] * ADOWN * invG * invV * invQ);
                    *reinterpret_cast<float2 *>(ov + db * 8 + 2 * tig) = make_float2(dv[db][2 * half] * ADOWN * invG, dv[db][2 * half + 1] * ADOWN * invG);
                }
            }
        }
    }
}

// --------------------------------------------------------------------------------------
// forward, whole tile resident: attn_fwd_tile_kernel (head_dim 32 or 64, float32 store).  Same staging, operand format and
// fragment addressing as attn_bwd_tile_kernel; one warp per 16 query rows (4 warps), online softmax over blocks of
// 16 keys, O += P V with V read through ldmatrix.trans.
// --------------------------------------------------------------------------------------
constexpr size_t fwd_tile_smem_bytes(int hd, int maxk) {
    return (size_t)(64 + 2 * maxk) * (size_t)(hd * 4) + (size_t)maxk * 8 + 32;
}

template <int HD, int MINB, typename KVT>
__global__ void __launch_bounds__(128, MINB)
attn_fwd_tile_kernel(const float *__restrict__ Q, const KVT *__restrict__ K, const KVT *__restrict__ V,
                     float *__restrict__ O, float *__restrict__ LSE, const int32_t *__restrict__ sub_end,
                     const int64_t *__restrict__ chain_off, const int32_t *__restrict__ chain_ids,
                     const int32_t *__restrict__ chain_end_all, int n, int H, float scale, int tile0, int maxk) {
    constexpr int M = 64, NT = 128, TILE_ROW_BYTES = HD * 4, KS = HD / 16, NDB = HD / 8, NCH = HD / 4;
    constexpr bool LP = sizeof(KVT) == 2;              // bfloat16 store: single fp16 products, no lo parts
    extern __shared__ __align__(128) unsigned char tile_smem_raw[];
    unsigned char *sQ = tile_smem_raw, *sK = sQ + M * TILE_ROW_BYTES, *sV = sK + (size_t)maxk * TILE_ROW_BYTES;
    int2 *s_meta = reinterpret_cast<int2 *>(sV + (size_t)maxk * TILE_ROW_BYTES);   // [maxk] {key id, key subtree end}
    uint32_t *s_max = reinterpret_cast<uint32_t *>(s_meta + maxk);                  // [3] max |x| of Q, K, V (float bits)

    const int t = blockIdx.x + tile0, h = blockIdx.y, tid = threadIdx.x;
    const int warp = tid >> 5, lane = tid & 31, g = lane >> 2, tig = lane & 3;
    const int D = H * HD, hoff = h * HD;
    const int i0 = t * M;
    const int nt = min(M, n - i0);
    const int64_t coff = chain_off[t];
    const int p = (int)(chain_off[t + 1] - coff);
    const int nkeys = p + nt;
    const int nkp = (nkeys + 15) & ~15;
    const int32_t *chain = chain_ids + coff;
    const int32_t *chain_end = chain_end_all + coff;

    // ---- stage 1: raw rows by cp.async ----
    if (tid < 3) s_max[tid] = 0u;
    constexpr int RSTEP = NT / NCH, OSTEP = RSTEP * TILE_ROW_BYTES;
    const TileLane L = tile_lane<HD>(tid);
#pragma unroll
    for (int u = 0; u < M / RSTEP; u++) {
        const int r = L.r0 + u * RSTEP, o = L.raw + u * OSTEP;
        if (r < nt) cp_async16(sQ + o, Q + (int64_t)(i0 + r) * D + hoff + L.c * 4);
        else *reinterpret_cast<float4 *>(sQ + o) = make_float4(0.f, 0.f, 0.f, 0.f);
    }
    constexpr int RSTEPK = NT / (HD / 8), OSTEPK = RSTEPK * TILE_ROW_BYTES;
    static_assert(NT % (HD / 8) == 0 && RSTEPK % 8 == 0, "a thread's key rows must share their swizzle term");
    const KvLane LK = kv_lane<HD>(tid);
    if constexpr (LP) {
        for (int r = LK.r0, o = LK.raw; r < nkp; r += RSTEPK, o += OSTEPK) {
            if (r < nkeys) {
                const int kid = r < p ? __ldg(chain + r) : i0 + (r - p);
                const int64_t off = (int64_t)kid * D + hoff + (tid % (HD / 8)) * 8;
                cp_async16(sK + o, K + off); cp_async16(sV + o, V + off);
            } else {
                *reinterpret_cast<uint4 *>(sK + o) = make_uint4(0u, 0u, 0u, 0u);
                *reinterpret_cast<uint4 *>(sV + o) = make_uint4(0u, 0u, 0u, 0u);
            }
        }
    } else {
        for (int r = L.r0, o = L.raw; r < nkp; r += RSTEP, o += OSTEP) {
            if (r < nkeys) {
                const int kid = r < p ? __ldg(chain + r) : i0 + (r - p);
                const int64_t off = (int64_t)kid * D + hoff + L.c * 4;
                cp_async16(sK + o, K + off); cp_async16(sV + o, V + off);
            } else {
                *reinterpret_cast<float4 *>(sK + o) = make_float4(0.f, 0.f, 0.f, 0.f);
                *reinterpret_cast<float4 *>(sV + o) = make_float4(0.f, 0.f, 0.f, 0.f);
            }
        }
    }
    cp_async_commit();
    for (int j = tid; j < nkp; j += NT) {
        int kid = 0x7fffffff, kend = 0;
        if (j < p) { kid = __ldg(chain + j); kend = __ldg(chain_end + j); }
        else if (j < nkeys) { kid = i0 + (j - p); kend = __ldg(sub_end + kid); }
        s_meta[j] = make_int2(kid, kend);
    }
    cp_async_wait_all();                 // this thread's own chunks have landed (pass A reads only those)

    // ---- stage 2 (pass A): maxima of |x| per tensor ----
    {
        float mq = 0.f, mk = 0.f, mv = 0.f;
#pragma unroll
        for (int u = 0; u < M / RSTEP; u++) mq = abs_max4(mq, *reinterpret_cast<const float4 *>(sQ + L.raw + u * OSTEP));
        if constexpr (LP) {
            for (int r = LK.r0, o = LK.raw; r < nkp; r += RSTEPK, o += OSTEPK) {
                mk = abs_max_bf16x8(mk, *reinterpret_cast<const uint4 *>(sK + o));
                mv = abs_max_bf16x8(mv, *reinterpret_cast<const uint4 *>(sV + o));
            }
        } else {
            for (int r = L.r0, o = L.raw; r < nkp; r += RSTEP, o += OSTEP) {
                mk = abs_max4(mk, *reinterpret_cast<const float4 *>(sK + o));
                mv = abs_max4(mv, *reinterpret_cast<const float4 *>(sV + o));
            }
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            mq = fmaxf(mq, __shfl_xor_sync(0xffffffffu, mq, o)); mk = fmaxf(mk, __shfl_xor_sync(0xffffffffu, mk, o));
            mv = fmaxf(mv, __shfl_xor_sync(0xffffffffu, mv, o));
        }
        if (lane == 0) {
            atomicMax(&s_max[0], __float_as_uint(mq)); atomicMax(&s_max[1], __float_as_uint(mk)); atomicMax(&s_max[2], __float_as_uint(mv));
        }
    }
    __syncthreads();
    float sclQ, invQ, sclK, invK, sclV, invV;
    pow2_scale(s_max[0], 0, sclQ, invQ); pow2_scale(s_max[1], 0, sclK, invK); pow2_scale(s_max[2], 0, sclV, invV);

    // ---- stage 3 (pass B): convert in place (Q rows two at a time through the two-plane helper) ----
#pragma unroll
    for (int u = 0; u < M / RSTEP; u += 2) tile_convert2(sQ, sQ + OSTEP, L, u * OSTEP, sclQ, sclQ);
    if constexpr (LP) {
        for (int r = LK.r0, o = 0; r < nkp; r += RSTEPK, o += OSTEPK) { kv_convert_bf16(sK, LK, o, sclK); kv_convert_bf16(sV, LK, o, sclV); }
    } else {
        for (int r = L.r0, o = 0; r < nkp; r += RSTEP, o += OSTEP) tile_convert2(sK, sV, L, o, sclK, sclV);
    }
    __syncthreads();

    const int rg = warp;
    if (rg * 16 >= nt) return;                                   // rows beyond the end of the plan (no barrier follows)
    const float fS = scale * LOG2E * invQ * invK;               // log2-domain score = S' * fS
    const int l8 = lane & 7, mi = lane >> 3;
    const uint32_t bRow = (uint32_t)(l8 * TILE_ROW_BYTES);
    const int bC = (mi & 1) + (mi >> 1) * NDB;
    const uint32_t aRow = (uint32_t)((l8 + (mi & 1) * 8) * TILE_ROW_BYTES);
    const int aC = mi >> 1, tC = (mi >> 1) * NDB;
    const uint32_t uQ = smem_u32_of(sQ), uK = smem_u32_of(sK), uV = smem_u32_of(sV);

    const int q0 = rg * 16 + g, q1 = q0 + 8;
    const int r0 = i0 + q0, r1 = i0 + q1;
    uint32_t qh[KS][4], ql[KS][4];
#pragma unroll
    for (int ks = 0; ks < KS; ks++) {
        const uint32_t o = (uint32_t)(rg * 16 * TILE_ROW_BYTES) + aRow;
        ldmatrix_x4(qh[ks], uQ + o + (uint32_t)(((2 * ks + aC) ^ l8) << 4));
        if constexpr (!LP) ldmatrix_x4(ql[ks], uQ + o + (uint32_t)(((2 * ks + aC + NDB) ^ l8) << 4));
    }
    float o_[NDB][4];
#pragma unroll
    for (int db = 0; db < NDB; db++) o_[db][0] = o_[db][1] = o_[db][2] = o_[db][3] = 0.f;
    float m0 = -INFINITY, m1 = -INFINITY, l0 = 0.f, l1 = 0.f;
    const int kp_lim = min((nkeys + 15) >> 4, (p + rg * 16 + 16 + 15) >> 4);
    for (int kp = 0; kp < kp_lim; kp++) {
        bool vld[2][4];
        bool on[2];
#pragma unroll
        for (int u = 0; u < 2; u++) {
            const int4 mk = *reinterpret_cast<const int4 *>(&s_meta[kp * 16 + u * 8 + 2 * tig]);
            vld[u][0] = mk.x <= r0 && r0 < mk.y; vld[u][1] = mk.z <= r0 && r0 < mk.w;
            vld[u][2] = mk.x <= r1 && r1 < mk.y; vld[u][3] = mk.z <= r1 && r1 < mk.w;
            on[u] = __any_sync(0xffffffffu, vld[u][0] | vld[u][1] | vld[u][2] | vld[u][3]);
        }
        if (!(on[0] || on[1])) continue;
        float s2[2][4];
#pragma unroll
        for (int u = 0; u < 2; u++) {
            s2[u][0] = s2[u][1] = s2[u][2] = s2[u][3] = -INFINITY;
            if (!on[u] && !TileBothHalves<HD>::fwd) continue;                  // warp-uniform
            float c[4] = {0.f, 0.f, 0.f, 0.f}, cx[4] = {0.f, 0.f, 0.f, 0.f};
            const uint32_t rowb = (uint32_t)((kp * 16 + u * 8) * TILE_ROW_BYTES) + bRow;
#pragma unroll
            for (int ks = 0; ks < KS; ks++) {
                uint32_t kf[4];
                ldmatrix_x4(kf, uK + rowb + (uint32_t)(((2 * ks + bC) ^ l8) << 4));
                mma_f16(c, qh[ks], kf[0], kf[1]);
                if constexpr (!LP) { mma_f16(cx, ql[ks], kf[0], kf[1]); mma_f16(cx, qh[ks], kf[2], kf[3]); }
            }
#pragma unroll
            for (int j = 0; j < 4; j++)
                if (vld[u][j]) s2[u][j] = fmaf(cx[j], LO_DOWN, c[j]) * fS;
        }
        float mx0 = fmaxf(fmaxf(s2[0][0], s2[0][1]), fmaxf(s2[1][0], s2[1][1]));
        float mx1 = fmaxf(fmaxf(s2[0][2], s2[0][3]), fmaxf(s2[1][2], s2[1][3]));
        mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1)); mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
        mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1)); mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
        const float mn0 = fmaxf(m0, mx0), mn1 = fmaxf(m1, mx1);
        const float mu0 = mn0 == -INFINITY ? 0.f : mn0, mu1 = mn1 == -INFINITY ? 0.f : mn1;
        // the running maxima of most rows stop moving after the first blocks: the rescaling (by exactly 1) is skipped then
        if (__any_sync(0xffffffffu, mn0 != m0 || mn1 != m1)) {
            const float corr0 = ex2_ftz(m0 - mu0), corr1 = ex2_ftz(m1 - mu1);
            l0 *= corr0; l1 *= corr1;
#pragma unroll
            for (int db = 0; db < NDB; db++) { o_[db][0] *= corr0; o_[db][1] *= corr0; o_[db][2] *= corr1; o_[db][3] *= corr1; }
        }
        m0 = mn0; m1 = mn1;
        float pw[2][4];
#pragma unroll
        for (int u = 0; u < 2; u++) {
            pw[u][0] = ex2_ftz(s2[u][0] - mu0); pw[u][1] = ex2_ftz(s2[u][1] - mu0);
            pw[u][2] = ex2_ftz(s2[u][2] - mu1); pw[u][3] = ex2_ftz(s2[u][3] - mu1);
            l0 += pw[u][0] + pw[u][1]; l1 += pw[u][2] + pw[u][3];
#pragma unroll
            for (int j = 0; j < 4; j++) pw[u][j] *= AUP;
        }
        uint32_t ph[4], pl[4], ps[4];
#pragma unroll
        for (int u = 0; u < 2; u++) {
            f16_split2<false>(pw[u][0], pw[u][1], ph[2 * u], pl[2 * u]); f16_split2<false>(pw[u][2], pw[u][3], ph[2 * u + 1], pl[2 * u + 1]);
            ps[2 * u] = f16_down11(ph[2 * u]); ps[2 * u + 1] = f16_down11(ph[2 * u + 1]);
        }
        const uint32_t rowt = uV + (uint32_t)(kp * 16 * TILE_ROW_BYTES) + aRow;
#pragma unroll
        for (int db = 0; db < NDB; db++) {
            uint32_t vt[4];                            // {b0 hi, b1 hi, b0 lo, b1 lo}: keys 0-7 / 8-15 of the block, dims 8 db..
            ldmatrix_x4_trans(vt, rowt + (uint32_t)(((db + tC) ^ l8) << 4));
            mma_f16(o_[db], ph, vt[0], vt[1]);
            if constexpr (!LP) { mma_f16(o_[db], pl, vt[0], vt[1]); mma_f16(o_[db], ps, vt[2], vt[3]); }
        }
    }
    l0 += __shfl_xor_sync(0xffffffffu, l0, 1); l0 += __shfl_xor_sync(0xffffffffu, l0, 2);
    l1 += __shfl_xor_sync(0xffffffffu, l1, 1); l1 += __shfl_xor_sync(0xffffffffu, l1, 2);
    if (r0 < n) {
        const float inv = ADOWN * invV / l0;
#pragma unroll
        for (int db = 0; db < NDB; db++)
            *reinterpret_cast<float2 *>(O + (int64_t)r0 * D + hoff + db * 8 + 2 * tig) = make_float2(o_[db][0] * inv, o_[db][1] * inv);
        if (tig == 0) LSE[(int64_t)r0 * H + h] = (m0 + log2f(l0)) * LN2;
    }
    if (r1 < n) {
        const float inv = ADOWN * invV / l1;
#pragma unroll
        for (int db = 0; db < NDB; db++)
            *reinterpret_cast<float2 *>(O + (int64_t)r1 * D + hoff + db * 8 + 2 * tig) = make_float2(o_[db][2] * inv, o_[db][3] * inv);
        if (tig == 0) LSE[(int64_t)r1 * H + h] = (m1 + log2f(l1)) * LN2;
    }
}

// dK/dV reduction, pass 1: one warp per work item = (node, tile range).  The node's row in tile t's
// partial block is chain_off[t] + depth - 1.  Tiles are summed in increasing order.
__global__ void reduce_items_kernel(const float *__restrict__ Pk, const float *__restrict__ Pv, float *__restrict__ dK,
                                    float *__restrict__ dV, float *__restrict__ segk, float *__restrict__ segv,
                                    const int64_t *__restrict__ chain_off, const int32_t *__restrict__ depth,
                                    const int32_t *__restrict__ item_node, const int32_t *__restrict__ item_t0,
                                    const int32_t *__restrict__ item_t1, const int32_t *__restrict__ item_slot,
                                    int64_t item0, int64_t n_items, int D) {
    int64_t it = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (it >= n_items) return;
    it += item0;
    const int lane = threadIdx.x & 31;
    const int a = item_node[it], t0 = item_t0[it], t1 = item_t1[it], slot = item_slot[it];
    const int row = depth[a] - 1;
    for (int c = lane * 4; c < D; c += 128) {
        float4 sk = make_float4(0.f, 0.f, 0.f, 0.f), sv = sk;
#pragma unroll 4
        for (int t = t0; t <= t1; t++) {
            int64_t r = (chain_off[t] + row) * D + c;
            float4 a4 = __ldcs(reinterpret_cast<const float4 *>(Pk + r));
            float4 b4 = __ldcs(reinterpret_cast<const float4 *>(Pv + r));
            sk.x += a4.x; sk.y += a4.y; sk.z += a4.z; sk.w += a4.w;
            sv.x += b4.x; sv.y += b4.y; sv.z += b4.z; sv.w += b4.w;
        }
        if (slot < 0) {
            float4 *pk = reinterpret_cast<float4 *>(dK + (int64_t)a * D + c), *pv = reinterpret_cast<float4 *>(dV + (int64_t)a * D + c);
            float4 x = *pk, y = *pv;
            *pk = make_float4(x.x + sk.x, x.y + sk.y, x.z + sk.z, x.w + sk.w);
            *pv = make_float4(y.x + sv.x, y.y + sv.y, y.z + sv.z, y.w + sv.w);
        } else {
            *reinterpret_cast<float4 *>(segk + (int64_t)slot * D + c) = sk;
            *reinterpret_cast<float4 *>(segv + (int64_t)slot * D + c) = sv;
        }
    }
}

// pass 2: nodes whose range was cut into several items; their segment sums are added in item order.
__global__ void reduce_multi_kernel(const float *__restrict__ segk, const float *__restrict__ segv, float *__restrict__ dK,
                                    float *__restrict__ dV, const int32_t *__restrict__ multi_node,
                                    const int32_t *__restrict__ multi_count, const int64_t *__restrict__ multi_first,
                                    const int32_t *__restrict__ item_slot, int64_t n_multi, int D) {
    int64_t mi = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (mi >= n_multi) return;
    const int lane = threadIdx.x & 31;
    const int a = multi_node[mi], cnt = multi_count[mi];
    const int slot0 = (int)multi_first[mi];           // slots of one node are consecutive
    (void)item_slot;
    for (int c = lane * 4; c < D; c += 128) {
        float4 sk = make_float4(0.f, 0.f, 0.f, 0.f), sv = sk;
        for (int s = 0; s < cnt; s++) {
            float4 a4 = *reinterpret_cast<const float4 *>(segk + (int64_t)(slot0 + s) * D + c);
            float4 b4 = *reinterpret_cast<const float4 *>(segv + (int64_t)(slot0 + s) * D + c);
            sk.x += a4.x; sk.y += a4.y; sk.z += a4.z; sk.w += a4.w;
            sv.x += b4.x; sv.y += b4.y; sv.z += b4.z; sv.w += b4.w;
        }
        float4 *pk = reinterpret_cast<float4 *>(dK + (int64_t)a * D + c), *pv = reinterpret_cast<float4 *>(dV + (int64_t)a * D + c);
        float4 x = *pk, y = *pv;
        *pk = make_float4(x.x + sk.x, x.y + sk.y, x.z + sk.z, x.w + sk.w);
        *pv = make_float4(y.x + sv.x, y.y + sv.y, y.z + sv.z, y.w + sv.w);
    }
}

// --------------------------------------------------------------------------------------
// native launchers
// --------------------------------------------------------------------------------------
static int check_common(const agpt_plan *p, int n_heads, int head_dim, const char *who) {
    if (!p) return agpt_set_error(AGPT_E_ARG, "%s: null plan", who);
    if (p->device < 0) return agpt_set_error(AGPT_E_ARG, "%s: plan has no device index (create it with device >= 0)", who);
    if (n_heads < 1 || n_heads > 65535) return agpt_set_error(AGPT_E_ARG, "%s: n_heads out of range", who);
    if (head_dim != 16 && head_dim != 32 && head_dim != 64)
        return agpt_set_error(AGPT_E_ARG, "%s: head_dim %d unsupported (16, 32 or 64)", who, head_dim);
    return AGPT_OK;
}

template <int HD, int M, typename KVT>
static int launch_fwd(const agpt_plan *p, const float *q, const void *k, const void *v, float *out, float *lse, int H,
                      float scale, cudaStream_t st, int tile0, int ntiles) {
    dim3 grid((unsigned)ntiles, (unsigned)H);
    attn_fwd_kernel<HD, M, KVT><<<grid, M, 0, st>>>(q, (const KVT *)k, (const KVT *)v, out, lse, p->d_sub_end,
                                                    p->d_chain_off, p->d_chain_ids, (int)p->n, H, scale, tile0);
    return launch_status("attn_fwd");
}

template <int HD, int M, typename KVT>
static int launch_bwd(const agpt_plan *p, const float *q, const void *k, const void *v, const float *o, const float *lse,
                      const float *dout, float *dq, float *dk, float *dv, float *pk, float *pv, int H, float scale,
                      cudaStream_t st, int tile0, int ntiles, BwdMask gmask) {
    dim3 grid((unsigned)ntiles, (unsigned)H);
    size_t smem = sizeof(BwdSmem<HD, M>);
    static size_t granted[AGPT_MAX_DEVICES];
    if (int rc = allow_dynamic_smem(attn_bwd_kernel<HD, M, KVT>, smem, granted)) return rc;
    attn_bwd_kernel<HD, M, KVT><<<grid, M, smem, st>>>(q, (const KVT *)k, (const KVT *)v, o, lse, dout, dq, dk, dv, pk, pv,
                                                       p->d_sub_end, p->d_chain_off, p->d_chain_ids, (int)p->n, H, scale, tile0, gmask);
    return launch_status("attn_bwd");
}

#define DISPATCH_HD_M_KV(FN, ...)                                                                  \
    do {                                                                                           \
        const bool bf = kv_dtype == AGPT_KV_BF16;                                                  \
        const int m_ = p->tile_m;                                                                  \
        if (head_dim == 16 && m_ == 32) return bf ? FN<16, 32, __nv_bfloat16>(__VA_ARGS__) : FN<16, 32, float>(__VA_ARGS__);   \
        if (head_dim == 16 && m_ == 64) return bf ? FN<16, 64, __nv_bfloat16>(__VA_ARGS__) : FN<16, 64, float>(__VA_ARGS__);   \
        if (head_dim == 16 && m_ == 128) return bf ? FN<16, 128, __nv_bfloat16>(__VA_ARGS__) : FN<16, 128, float>(__VA_ARGS__); \
        if (head_dim == 32 && m_ == 32) return bf ? FN<32, 32, __nv_bfloat16>(__VA_ARGS__) : FN<32, 32, float>(__VA_ARGS__);   \
        if (head_dim == 32 && m_ == 64) return bf ? FN<32, 64, __nv_bfloat16>(__VA_ARGS__) : FN<32, 64, float>(__VA_ARGS__);   \
        if (head_dim == 32 && m_ == 128) return bf ? FN<32, 128, __nv_bfloat16>(__VA_ARGS__) : FN<32, 128, float>(__VA_ARGS__); \
        if (head_dim == 64 && m_ == 32) return bf ? FN<64, 32, __nv_bfloat16>(__VA_ARGS__) : FN<64, 32, float>(__VA_ARGS__);   \
        if (head_dim == 64 && m_ == 64) return bf ? FN<64, 64, __nv_bfloat16>(__VA_ARGS__) : FN<64, 64, float>(__VA_ARGS__);   \
        if (head_dim == 64 && m_ == 128) return bf ? FN<64, 128, __nv_bfloat16>(__VA_ARGS__) : FN<64, 128, float>(__VA_ARGS__); \
        return agpt_set_error(AGPT_E_ARG, "unsupported head_dim/tile combination");               \
    } while (0)

// Kernel family of the native attention entry points: 1 = tensor cores (mma.sync TF32, error-compensated; tiles
// of 64), 0 = FP32 FMA.  Initialised from the environment variable AGPT_B200_ATTN_IMPL, default 1.
static int g_attn_impl = -1;
static int attn_impl() {
    if (g_attn_impl < 0) {
        const char *e = getenv("AGPT_B200_ATTN_IMPL");
        g_attn_impl = (e && e[0] == '0') ? 0 : 1;
    }
    return g_attn_impl;
}
extern "C" int agpt_b200_set_attn_impl(int impl) {
    if (impl != 0 && impl != 1) return agpt_set_error(AGPT_E_ARG, "set_attn_impl: 0 (FMA) or 1 (tensor cores)");
    g_attn_impl = impl;
    return AGPT_OK;
}

// Whole-tile kernels (forward and backward; float32 store, head_dim 32): chosen when four blocks of the backward
// fit one SM (228 KB of shared memory, 1 KB reserved per block), i.e. up to about 150 keys per tile; deeper plans take
// the chunked kernels.  AGPT_B200_ATTN_TILE=0 keeps the chunked kernels (A/B runs); AGPT_B200_BWD_WARPS = 4, 6 or 8
// warps per block of the backward.
// head_dim 32: four blocks of the backward per SM; head_dim 64 (rows twice as long, twice the registers): two
static inline bool tile_kernels_fit(const agpt_plan *p, int head_dim);
static int g_bwd_tile = -1, g_bwd_warps = 0, g_bwd_dbg = 0;
static int bwd_tile_enabled() {
    if (g_bwd_tile < 0) {
        const char *e = getenv("AGPT_B200_ATTN_TILE");
        g_bwd_tile = (e && e[0] == '0') ? 0 : 1;
        const char *w = getenv("AGPT_B200_BWD_WARPS");
        g_bwd_warps = w ? atoi(w) : 4;
        const char *d = getenv("AGPT_B200_BWD_DEBUG");
        g_bwd_dbg = d ? atoi(d) : 0;
        if (g_bwd_warps != 3 && g_bwd_warps != 6 && g_bwd_warps != 8) g_bwd_warps = 4;
    }
    return g_bwd_tile;
}
extern "C" int agpt_b200_set_attn_variant(int whole_tile, int warps) {
    if ((whole_tile != 0 && whole_tile != 1) || (warps != 3 && warps != 4 && warps != 6 && warps != 8))
        return agpt_set_error(AGPT_E_ARG, "set_attn_variant: whole_tile 0 or 1, bwd_warps 4, 6 or 8");
    bwd_tile_enabled();
    g_bwd_tile = whole_tile; g_bwd_warps = warps;
    return AGPT_OK;
}
static inline int bwd_tile_maxk(const agpt_plan *p) { return ((p->max_depth - 1 + 64) + 15) & ~15; }
static inline bool tile_kernels_fit(const agpt_plan *p, int head_dim) {
    if (head_dim != 32 && head_dim != 64) return false;
    return bwd_tile_smem_bytes(head_dim, bwd_tile_maxk(p)) <= (head_dim == 32 ? (size_t)56 * 1024 : (size_t)113 * 1024);
}
// Whole-tile backward for a bfloat16 store (AGPT_B200_ATTN_TILE_BF16=0: the chunked kernel, which keeps float32-level
// products).  Measured: head_dim 32 (depth-32 trie, 28.3M positions) 42.3 ms against 45.5 ms chunked; head_dim 64 (4M-node
// tree) 29.4 ms against 26.8 ms, so head_dim 64 stays chunked; the forward is no faster either way (15.1 ms) and stays chunked.
static int tile_bf16_enabled() {
    static int on = -1;
    if (on < 0) {
        const char *e = getenv("AGPT_B200_ATTN_TILE_BF16");
        on = (e && e[0] == '0') ? 0 : 1;
    }
    return on;
}

template <int HD, int MINB, typename KVT>
static int launch_fwd_tile(const agpt_plan *p, const float *q, const void *k, const void *v, float *out, float *lse, int H,
                           float scale, cudaStream_t st, int tile0, int ntiles) {
    static size_t granted[AGPT_MAX_DEVICES];
    const int maxk = bwd_tile_maxk(p);
    const size_t smem = fwd_tile_smem_bytes(HD, maxk);
    int rc = allow_dynamic_smem(attn_fwd_tile_kernel<HD, MINB, KVT>, smem, granted);
    if (rc) return rc;
    dim3 grid((unsigned)ntiles, (unsigned)H);
    attn_fwd_tile_kernel<HD, MINB, KVT><<<grid, 128, smem, st>>>(q, (const KVT *)k, (const KVT *)v, out, lse, p->d_sub_end,
                                                                 p->d_chain_off, p->d_chain_ids, p->d_chain_end, (int)p->n, H, scale, tile0, maxk);
    return launch_status("attn_fwd_tile");
}

template <int HD, typename KVT>
static int launch_fwd_mma(const agpt_plan *p, const float *q, const void *k, const void *v, float *out, float *lse, int H,
                          float scale, cudaStream_t st, int tile0, int ntiles) {
    dim3 grid((unsigned)ntiles, (unsigned)H);
    const size_t smem = fwd_mma_smem_bytes<HD>();
    static size_t granted[AGPT_MAX_DEVICES];
    if (int rc = allow_dynamic_smem(attn_fwd_mma_kernel<HD, KVT>, smem, granted)) return rc;
    attn_fwd_mma_kernel<HD, KVT><<<grid, 128, smem, st>>>(q, (const KVT *)k, (const KVT *)v, out, lse, p->d_sub_end,
                                                       p->d_chain_off, p->d_chain_ids, p->d_chain_end, (int)p->n, H, scale, tile0);
    return launch_status("attn_fwd_mma");
}

static int fwd_dispatch(const agpt_plan *p, const float *q, const void *k, const void *v, int kv_dtype, float *out,
                        float *lse, int H, int head_dim, float scale, cudaStream_t st, int tile0, int ntiles) {
    // head_dim 64: the whole-tile forward (two blocks per SM) measured slower than the chunked one (17.5 vs 15.0 ms on the
    // 4M-node microbenchmark), the whole-tile backward faster (37.7 vs 50.3 ms): the forward stays chunked there
    if (attn_impl() == 1 && p->tile_m == 64 && kv_dtype == AGPT_KV_F32 && head_dim == 32 && bwd_tile_enabled() && tile_kernels_fit(p, head_dim))
    {
        // six blocks of four warps per SM (80 registers, no spills; the 33.6 KB of a depth-32 tile fit six times): 19.0 ms on
        // the depth-32 trie against 20.1 ms with five (95 registers; AGPT_B200_FWD_BLOCKS=5).  The backward does not gain
        // from a fifth block (96 registers with spills: 52.5 against 49.9 ms).
        static int blocks = 0;
        if (!blocks) { const char *e = getenv("AGPT_B200_FWD_BLOCKS"); blocks = (e && atoi(e) == 5) ? 5 : 6; }
        if (blocks == 6) return launch_fwd_tile<32, 6, float>(p, q, k, v, out, lse, H, scale, st, tile0, ntiles);
        return launch_fwd_tile<32, 5, float>(p, q, k, v, out, lse, H, scale, st, tile0, ntiles);
    }
    if (attn_impl() == 1 && p->tile_m == 64 && p->max_depth + 64 <= MAXKEYS) {
        const bool bf = kv_dtype == AGPT_KV_BF16;
        switch (head_dim) {
            case 16: return bf ? launch_fwd_mma<16, __nv_bfloat16>(p, q, k, v, out, lse, H, scale, st, tile0, ntiles) : launch_fwd_mma<16, float>(p, q, k, v, out, lse, H, scale, st, tile0, ntiles);
            case 32: return bf ? launch_fwd_mma<32, __nv_bfloat16>(p, q, k, v, out, lse, H, scale, st, tile0, ntiles) : launch_fwd_mma<32, float>(p, q, k, v, out, lse, H, scale, st, tile0, ntiles);
            case 64: return bf ? launch_fwd_mma<64, __nv_bfloat16>(p, q, k, v, out, lse, H, scale, st, tile0, ntiles) : launch_fwd_mma<64, float>(p, q, k, v, out, lse, H, scale, st, tile0, ntiles);
        }
    }
    DISPATCH_HD_M_KV(launch_fwd, p, q, k, v, out, lse, H, scale, st, tile0, ntiles);
}

template <int HD, typename KVT>
static int launch_bwd_mma(const agpt_plan *p, const float *q, const void *k, const void *v, const float *o, const float *lse,
                          const float *dout, float *dq, float *dk, float *dv, float *pk, float *pv, int H, float scale,
                          cudaStream_t st, int tile0, int ntiles, BwdMask gmask) {
    dim3 grid((unsigned)ntiles, (unsigned)H);
    size_t smem = sizeof(BwdMmaSmem<HD, KVT>);
    static size_t granted[AGPT_MAX_DEVICES];
    if (int rc = allow_dynamic_smem(attn_bwd_mma_kernel<HD, KVT>, smem, granted)) return rc;
    attn_bwd_mma_kernel<HD, KVT><<<grid, 128, smem, st>>>(q, (const KVT *)k, (const KVT *)v, o, lse, dout, dq, dk, dv, pk, pv,
                                                          p->d_sub_end, p->d_chain_off, p->d_chain_ids, p->d_chain_end, (int)p->n, H,
                                                          scale, tile0, gmask);
    return launch_status("attn_bwd_mma");
}

template <int HD, int NW, int MINB, typename KVT = float>
static int launch_bwd_tile(const agpt_plan *p, const float *q, const void *k, const void *v, const float *o, const float *lse,
                           const float *dout, float *dq, float *dk, float *dv, float *pk, float *pv, int H, float scale,
                           cudaStream_t st, int tile0, int ntiles, BwdMask gmask) {
    static size_t granted[AGPT_MAX_DEVICES];
    const int maxk = bwd_tile_maxk(p);
    const size_t smem = bwd_tile_smem_bytes(HD, maxk);
    int rc = allow_dynamic_smem(attn_bwd_tile_kernel<HD, NW, MINB, KVT>, smem, granted);
    if (rc) return rc;
    dim3 grid((unsigned)ntiles, (unsigned)H);
    attn_bwd_tile_kernel<HD, NW, MINB, KVT><<<grid, NW * 32, smem, st>>>(q, (const KVT *)k, (const KVT *)v, o, lse, dout, dq, dk, dv, pk, pv,
                                                                         p->d_sub_end, p->d_chain_off, p->d_chain_ids, p->d_chain_end,
                                                                         (int)p->n, H, scale, tile0, maxk, g_bwd_dbg, gmask);
    return launch_status("attn_bwd_tile");
}

static int launch_bwd_tile_w(const agpt_plan *p, const float *q, const void *k, const void *v, int kv_dtype, const float *o,
                             const float *lse, const float *dout, float *dq, float *dk, float *dv, float *pk, float *pv, int H,
                             int head_dim, float scale, cudaStream_t st, int tile0, int ntiles, BwdMask gmask) {
#define TILE_ARGS p, q, k, v, o, lse, dout, dq, dk, dv, pk, pv, H, scale, st, tile0, ntiles, gmask
    if (kv_dtype == AGPT_KV_BF16) return launch_bwd_tile<32, 4, 4, __nv_bfloat16>(TILE_ARGS);    // head_dim 32 only (bwd_dispatch)
    if (head_dim == 64) {        // twice the fragment and accumulator registers: two blocks per SM
        switch (g_bwd_warps) {
            case 6: case 8: return launch_bwd_tile<64, 8, 1>(TILE_ARGS);
            default: return launch_bwd_tile<64, 4, 2>(TILE_ARGS);
        }
    }
    switch (g_bwd_warps) {
        case 3: return launch_bwd_tile<32, 4, 3>(TILE_ARGS);
        case 6: return launch_bwd_tile<32, 6, 3>(TILE_ARGS);
        case 8: return launch_bwd_tile<32, 8, 2>(TILE_ARGS);
        default: return launch_bwd_tile<32, 4, 4>(TILE_ARGS);
    }
#undef TILE_ARGS
}

static int bwd_dispatch(const agpt_plan *p, const float *q, const void *k, const void *v, int kv_dtype, const float *o,
                        const float *lse, const float *dout, float *dq, float *dk, float *dv, float *pk, float *pv, int H,
                        int head_dim, float scale, cudaStream_t st, int tile0, int ntiles, BwdMask gmask = BwdMask{AGPT_GRAD_FULL, nullptr}) {
    if (attn_impl() == 1 && p->tile_m == 64 && bwd_tile_enabled() &&
        (kv_dtype == AGPT_KV_F32 || (head_dim == 32 && tile_bf16_enabled()))) {
        if (tile_kernels_fit(p, head_dim))
            return launch_bwd_tile_w(p, q, k, v, kv_dtype, o, lse, dout, dq, dk, dv, pk, pv, H, head_dim, scale, st, tile0, ntiles, gmask);
    }
    if (attn_impl() == 1 && p->tile_m == 64 && p->max_depth + 64 <= MAXKEYS) {
        const bool bf = kv_dtype == AGPT_KV_BF16;
#define BWD_MMA_ARGS p, q, k, v, o, lse, dout, dq, dk, dv, pk, pv, H, scale, st, tile0, ntiles, gmask
        switch (head_dim) {
            case 16: return bf ? launch_bwd_mma<16, __nv_bfloat16>(BWD_MMA_ARGS) : launch_bwd_mma<16, float>(BWD_MMA_ARGS);
            case 32: return bf ? launch_bwd_mma<32, __nv_bfloat16>(BWD_MMA_ARGS) : launch_bwd_mma<32, float>(BWD_MMA_ARGS);
            case 64: return bf ? launch_bwd_mma<64, __nv_bfloat16>(BWD_MMA_ARGS) : launch_bwd_mma<64, float>(BWD_MMA_ARGS);
        }
#undef BWD_MMA_ARGS
    }
    DISPATCH_HD_M_KV(launch_bwd, p, q, k, v, o, lse, dout, dq, dk, dv, pk, pv, H, scale, st, tile0, ntiles, gmask);
}

extern "C" int agpt_b200_attn_fwd(const agpt_plan *p, const float *d_q, const void *d_k, const void *d_v, int kv_dtype,
                                  float *d_out, float *d_lse, int n_heads, int head_dim, float scale, void *stream) {
    int rc = check_common(p, n_heads, head_dim, "attn_fwd");
    if (rc) return rc;
    if (!d_q || !d_k || !d_v || !d_out || !d_lse) return agpt_set_error(AGPT_E_ARG, "attn_fwd: null buffer");
    if (kv_dtype != AGPT_KV_F32 && kv_dtype != AGPT_KV_BF16) return agpt_set_error(AGPT_E_ARG, "attn_fwd: bad kv_dtype");
    return fwd_dispatch(p, d_q, d_k, d_v, kv_dtype, d_out, d_lse, n_heads, head_dim, scale, (cudaStream_t)stream, 0, (int)p->n_tiles);
}

// Reduction pass 1 over items [item0, item1) (the list is ordered by last tile), then, if requested, pass 2.
static int run_reduce_range(const agpt_plan *p, float *pk, float *pv, float *segk, float *segv, float *dk, float *dv, int D,
                            cudaStream_t st, int64_t item0, int64_t item1, bool multi_pass) {
    const int64_t n_items = item1 - item0;
    if (n_items > 0) {
        const int wpb = 8;
        reduce_items_kernel<<<(unsigned)((n_items + wpb - 1) / wpb), wpb * 32, 0, st>>>(
            pk, pv, dk, dv, segk, segv, p->d_chain_off, p->d_depth, p->d_item_node, p->d_item_t0, p->d_item_t1,
            p->d_item_slot, item0, n_items, D);
        int rc = launch_status("reduce_items");
        if (rc) return rc;
    }
    int64_t n_multi = (int64_t)p->multi_node.size();
    if (multi_pass && n_multi > 0) {
        const int wpb = 4;
        reduce_multi_kernel<<<(unsigned)((n_multi + wpb - 1) / wpb), wpb * 32, 0, st>>>(
            segk, segv, dk, dv, p->d_multi_node, p->d_multi_count, p->d_multi_first, p->d_item_slot, n_multi, D);
        int rc = launch_status("reduce_multi");
        if (rc) return rc;
    }
    return AGPT_OK;
}

static int run_reduce(const agpt_plan *p, float *pk, float *pv, float *segk, float *segv, float *dk, float *dv, int D,
                      cudaStream_t st) {
    return run_reduce_range(p, pk, pv, segk, segv, dk, dv, D, st, 0, (int64_t)p->item_node.size(), true);
}

extern "C" int agpt_b200_attn_bwd_mode(const agpt_plan *p, const float *d_q, const void *d_k, const void *d_v, int kv_dtype,
                                       const float *d_out, const float *d_lse, const float *d_dout, float *d_dq, float *d_dk,
                                       float *d_dv, void *d_workspace, int64_t workspace_bytes, int n_heads, int head_dim,
                                       float scale, int grad_mode, const int32_t *d_edge_first, void *stream) {
    int rc = check_common(p, n_heads, head_dim, "attn_bwd");
    if (rc) return rc;
    if (!d_q || !d_k || !d_v || !d_out || !d_lse || !d_dout || !d_dq || !d_dk || !d_dv || !d_workspace)
        return agpt_set_error(AGPT_E_ARG, "attn_bwd: null buffer");
    if (kv_dtype != AGPT_KV_F32 && kv_dtype != AGPT_KV_BF16) return agpt_set_error(AGPT_E_ARG, "attn_bwd: bad kv_dtype");
    if (grad_mode != AGPT_GRAD_FULL && grad_mode != AGPT_GRAD_LOCAL_DEPTH && grad_mode != AGPT_GRAD_OWN_EDGE)
        return agpt_set_error(AGPT_E_ARG, "attn_bwd: grad_mode %d unknown", grad_mode);
    if (grad_mode == AGPT_GRAD_OWN_EDGE && !d_edge_first)
        return agpt_set_error(AGPT_E_ARG, "attn_bwd: the own-edge mode needs the edge_first array");
    const int D = n_heads * head_dim;
    int64_t need = agpt_b200_attn_bwd_workspace_bytes(p, D);
    if (workspace_bytes < need)
        return agpt_set_error(AGPT_E_ARG, "attn_bwd: workspace %lld bytes < required %lld", (long long)workspace_bytes, (long long)need);
    const int64_t rows = (int64_t)p->chain_ids.size();
    float *pk = (float *)d_workspace, *pv = pk + rows * D, *segk = pv + rows * D, *segv = segk + p->n_multi_items * D;
    rc = bwd_dispatch(p, d_q, d_k, d_v, kv_dtype, d_out, d_lse, d_dout, d_dq, d_dk, d_dv, pk, pv, n_heads, head_dim, scale,
                      (cudaStream_t)stream, 0, (int)p->n_tiles, BwdMask{grad_mode, d_edge_first});
    if (rc) return rc;
    return run_reduce(p, pk, pv, segk, segv, d_dk, d_dv, D, (cudaStream_t)stream);
}

extern "C" int agpt_b200_attn_bwd(const agpt_plan *p, const float *d_q, const void *d_k, const void *d_v, int kv_dtype,
                                  const float *d_out, const float *d_lse, const float *d_dout, float *d_dq, float *d_dk,
                                  float *d_dv, void *d_workspace, int64_t workspace_bytes, int n_heads, int head_dim,
                                  float scale, void *stream) {
    return agpt_b200_attn_bwd_mode(p, d_q, d_k, d_v, kv_dtype, d_out, d_lse, d_dout, d_dq, d_dk, d_dv, d_workspace, workspace_bytes,
                                   n_heads, head_dim, scale, AGPT_GRAD_FULL, nullptr, stream);
}

// --------------------------------------------------------------------------------------
// row gather, RoPE, bf16 store write
// --------------------------------------------------------------------------------------
__global__ void gather_rows_kernel(const float *__restrict__ src, const int32_t *__restrict__ index, float *__restrict__ dst,
                                   int64_t n, int cols4) {
    int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= n * cols4) return;
    int64_t r = idx / cols4;
    int c = (int)(idx % cols4);
    reinterpret_cast<float4 *>(dst)[idx] = __ldg(reinterpret_cast<const float4 *>(src) + (int64_t)index[r] * cols4 + c);
}

extern "C" int agpt_b200_gather_rows(const float *d_src, const int32_t *d_index, float *d_dst, int64_t n, int cols, void *stream) {
    if (!d_src || !d_index || !d_dst || n < 0 || cols <= 0 || cols % 4) return agpt_set_error(AGPT_E_ARG, "gather_rows: bad argument (cols must be a multiple of 4)");
    if (n == 0) return AGPT_OK;
    int64_t total = n * (cols / 4);
    gather_rows_kernel<<<(unsigned)((total + 255) / 256), 256, 0, (cudaStream_t)stream>>>(d_src, d_index, d_dst, n, cols / 4);
    return launch_status("gather_rows");
}

__global__ void rope_kernel(float *__restrict__ x, const int32_t *__restrict__ pos, const float *__restrict__ cosv,
                            const float *__restrict__ sinv, int64_t n, int H, int hd, int inverse) {
    const int half = hd / 2;
    int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= n * H * half) return;
    int64_t row = idx / (H * half);
    int rem = (int)(idx % (H * half));
    int h = rem / half, i = rem % half;
    int ps = pos[row];
    float c = cosv[ps * hd + 2 * i], s = sinv[ps * hd + 2 * i];
    float2 *px = reinterpret_cast<float2 *>(x + row * (int64_t)(H * hd) + h * hd + 2 * i);
    float2 v = *px;
    if (!inverse) *px = make_float2(v.x * c - v.y * s, v.x * s + v.y * c);
    else *px = make_float2(v.x * c + v.y * s, -v.x * s + v.y * c);
}

// Four columns (two rotation pairs) per thread and step, ROPE_ROWS rows per block, one or two matrices that share
// the row positions (q and k, or dq and dk): every thread has several independent 16-byte loads in flight and the
// position and table reads are shared between the two matrices.
#define ROPE_ROWS 32
template <bool TWO>
__global__ void __launch_bounds__(256)
rope4_kernel(float *a, float *b, const int32_t *__restrict__ pos, const float *__restrict__ cosv, const float *__restrict__ sinv,
             int64_t n, int D, int hd, int inverse) {
    const int q4n = D >> 2;
    const int64_t row0 = (int64_t)blockIdx.x * ROPE_ROWS;
    const int rows = (int)(n - row0 < ROPE_ROWS ? n - row0 : ROPE_ROWS);
    const float sign = inverse ? -1.f : 1.f;
    for (int t = threadIdx.x; t < rows * q4n; t += 256) {
        const int r = t / q4n, c = (t - r * q4n) << 2;
        const int64_t off = (row0 + r) * D + c;
        const int tab = __ldg(pos + row0 + r) * hd + (c % hd);
        const float4 cs = __ldg(reinterpret_cast<const float4 *>(cosv + tab));
        float4 sn = __ldg(reinterpret_cast<const float4 *>(sinv + tab));
        sn.x *= sign; sn.z *= sign;
        float4 v = __ldcs(reinterpret_cast<const float4 *>(a + off));
        __stcs(reinterpret_cast<float4 *>(a + off),
               make_float4(v.x * cs.x - v.y * sn.x, v.x * sn.x + v.y * cs.x, v.z * cs.z - v.w * sn.z, v.z * sn.z + v.w * cs.z));
        if (TWO) {
            v = __ldcs(reinterpret_cast<const float4 *>(b + off));
            __stcs(reinterpret_cast<float4 *>(b + off),
                   make_float4(v.x * cs.x - v.y * sn.x, v.x * sn.x + v.y * cs.x, v.z * cs.z - v.w * sn.z, v.z * sn.z + v.w * cs.z));
        }
    }
}

static int rope_launch(float *d_a, float *d_b, const int32_t *d_pos, const float *d_cos, const float *d_sin, int64_t n, int n_heads,
                       int head_dim, int inverse, cudaStream_t st) {
    if (!d_a || !d_pos || !d_cos || !d_sin || n < 0 || n_heads < 1 || head_dim < 2 || head_dim % 2)
        return agpt_set_error(AGPT_E_ARG, "rope: bad argument");
    if (n == 0) return AGPT_OK;
    const bool vec = head_dim % 4 == 0 && (((uintptr_t)d_a | (uintptr_t)d_b | (uintptr_t)d_cos | (uintptr_t)d_sin) & 15) == 0;
    if (vec) {
        const unsigned blocks = (unsigned)((n + ROPE_ROWS - 1) / ROPE_ROWS);
        if (d_b) rope4_kernel<true><<<blocks, 256, 0, st>>>(d_a, d_b, d_pos, d_cos, d_sin, n, n_heads * head_dim, head_dim, inverse);
        else rope4_kernel<false><<<blocks, 256, 0, st>>>(d_a, nullptr, d_pos, d_cos, d_sin, n, n_heads * head_dim, head_dim, inverse);
        return launch_status("rope");
    }
    int64_t total = n * n_heads * (head_dim / 2);
    rope_kernel<<<(unsigned)((total + 255) / 256), 256, 0, st>>>(d_a, d_pos, d_cos, d_sin, n, n_heads, head_dim, inverse);
    if (d_b) rope_kernel<<<(unsigned)((total + 255) / 256), 256, 0, st>>>(d_b, d_pos, d_cos, d_sin, n, n_heads, head_dim, inverse);
    return launch_status("rope");
}

extern "C" int agpt_b200_rope(float *d_x, const int32_t *d_pos, const float *d_cos, const float *d_sin, int64_t n, int n_heads,
                              int head_dim, int inverse, void *stream) {
    return rope_launch(d_x, nullptr, d_pos, d_cos, d_sin, n, n_heads, head_dim, inverse, (cudaStream_t)stream);
}

extern "C" int agpt_b200_rope_pair(float *d_a, float *d_b, const int32_t *d_pos, const float *d_cos, const float *d_sin, int64_t n,
                                   int n_heads, int head_dim, int inverse, void *stream) {
    if (!d_b) return agpt_set_error(AGPT_E_ARG, "rope_pair: bad argument");
    return rope_launch(d_a, d_b, d_pos, d_cos, d_sin, n, n_heads, head_dim, inverse, (cudaStream_t)stream);
}

__global__ void store_bf16_kernel(const float *__restrict__ src, __nv_bfloat16 *__restrict__ dst, int64_t total4) {
    int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= total4) return;
    float4 v = __ldg(reinterpret_cast<const float4 *>(src) + idx);
    __nv_bfloat162 a = __floats2bfloat162_rn(v.x, v.y), b = __floats2bfloat162_rn(v.z, v.w);
    uint2 o;
    o.x = *reinterpret_cast<uint32_t *>(&a); o.y = *reinterpret_cast<uint32_t *>(&b);
    reinterpret_cast<uint2 *>(dst)[idx] = o;
}

extern "C" int agpt_b200_kv_store_write_bf16(const float *d_src, void *d_store, int64_t n, int cols, void *stream) {
    if (!d_src || !d_store || n < 0 || cols <= 0 || cols % 4) return agpt_set_error(AGPT_E_ARG, "kv_store_write_bf16: bad argument");
    if (n == 0) return AGPT_OK;
    int64_t total4 = n * (cols / 4);
    store_bf16_kernel<<<(unsigned)((total4 + 255) / 256), 256, 0, (cudaStream_t)stream>>>(d_src, (__nv_bfloat16 *)d_store, total4);
    return launch_status("kv_store_write_bf16");
}

// --------------------------------------------------------------------------------------
// loss: one warp per query row
// --------------------------------------------------------------------------------------
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ int warp_sum_i(int v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

// mode 0: per-query (radix); mode 1: per-node (leveled, node_ids index the counts).
// One warp per batch of 32 consecutive rows.  The index loads of a row form a dependent chain (query -> node ->
// offsets -> counts) several memory latencies long; lane l walks the chain of row l of the batch, so the 32 chains
// are in flight together and their loads coalesce, and the row loop then takes each row's indices from its lane
// by shuffle.  The logits of row k+1 are requested before row k is reduced.  NPL > 0: a row (V <= 32*NPL) lives
// in registers, lane l owning columns l, l+32, ...; shared memory is touched only by rows that end a radix edge
// (sparse count lookups).  NPL == 0: any V, the row lives in shared memory.  Either way every logit is read once,
// exponentiated once, and every gradient element written once.
#define LOSS_WPB 8
#define LOSS_ROWS_PER_BLOCK (LOSS_WPB * 32)
template <int NPL>
__global__ void __launch_bounds__(LOSS_WPB * 32, 8)
loss_kernel(const float *__restrict__ logits, const int32_t *__restrict__ query_to_node,
            const int32_t *__restrict__ query_offsets, const int32_t *__restrict__ ids,
            const int32_t *__restrict__ token_ids, const int32_t *__restrict__ counts_offset,
            const int32_t *__restrict__ counts_tok, const int32_t *__restrict__ counts_val,
            const float *__restrict__ mass_weights, float *__restrict__ d_logits, float *__restrict__ loss_out,
            int64_t T_q, int V, float entropy_lambda, float intermediate_weight, int ce_only, int mode) {
    extern __shared__ float s_rows[];
    const int64_t r0 = ((int64_t)blockIdx.x * LOSS_WPB + (threadIdx.x >> 5)) * 32;
    if (r0 >= T_q) return;
    const int nrows = (T_q - r0 < 32) ? (int)(T_q - r0) : 32;
    const int lane = threadIdx.x & 31;
    float *row = s_rows + (threadIdx.x >> 5) * V;
    constexpr int NR = NPL > 0 ? NPL : 1;
    constexpr float NEG = -3.402823466e+38f;

    // lane-parallel index chains of the batch
    int my_ep = 0, my_target = 0, my_cs = 0, my_ce = 0;
    float my_mw = 1.0f;
    if (lane < nrows) {
        const int64_t qi = r0 + lane;
        bool endpoint_path;
        int cid = 0;
        if (mode == 1) { endpoint_path = true; cid = ids[qi]; }
        else {
            int n_idx = query_to_node[qi];
            bool is_endpoint = (qi + 1) == query_offsets[n_idx + 1];
            bool ce_as_intermediate = ce_only && is_endpoint && (qi + 1 < T_q);
            endpoint_path = is_endpoint && !ce_as_intermediate;
            if (endpoint_path) cid = ids[n_idx];
        }
        if (endpoint_path) { my_cs = counts_offset[cid]; my_ce = counts_offset[cid + 1]; }
        else my_target = token_ids[qi + 1];
        if (mode == 0 && mass_weights) my_mw = mass_weights[qi];
        my_ep = endpoint_path ? 1 : 0;
    }

    float xn[NR];
    if (NPL > 0) {
#pragma unroll
        for (int k = 0; k < NR; k++) { const int j = lane + 32 * k; xn[k] = j < V ? __ldcs(logits + r0 * V + j) : NEG; }
    }
    for (int rr = 0; rr < nrows; rr++) {
        const int64_t qi = r0 + rr;
        const float *in = logits + qi * V;
        float *g = d_logits + qi * V;
        const bool endpoint_path = __shfl_sync(0xffffffffu, my_ep, rr) != 0;
        const int c_start = __shfl_sync(0xffffffffu, my_cs, rr), c_end = __shfl_sync(0xffffffffu, my_ce, rr);
        int target = __shfl_sync(0xffffffffu, my_target, rr);
        const float mass_w = __shfl_sync(0xffffffffu, my_mw, rr);
        float x[NR];
        float mx = NEG, sum = 0.f;
        if (NPL > 0) {
#pragma unroll
            for (int k = 0; k < NR; k++) { x[k] = xn[k]; mx = fmaxf(mx, x[k]); }
            if (rr + 1 < nrows) {
#pragma unroll
                for (int k = 0; k < NR; k++) { const int j = lane + 32 * k; xn[k] = j < V ? __ldcs(in + V + j) : NEG; }
            }
            mx = warp_max(mx);
#pragma unroll
            for (int k = 0; k < NR; k++) { x[k] = lane + 32 * k < V ? expf(x[k] - mx) : 0.f; sum += x[k]; }
            sum = warp_sum(sum);
            const float inv = 1.0f / sum;
#pragma unroll
            for (int k = 0; k < NR; k++) x[k] *= inv;                  // probabilities
        } else {
            for (int j = lane; j < V; j += 32) { float v = __ldcs(in + j); row[j] = v; mx = fmaxf(mx, v); }
            mx = warp_max(mx);
            for (int j = lane; j < V; j += 32) { float e = expf(row[j] - mx); row[j] = e; sum += e; }
            sum = warp_sum(sum);
            const float inv = 1.0f / sum;
            for (int j = lane; j < V; j += 32) row[j] *= inv;
            __syncwarp();
        }
        // probability of one column, the same for every lane
        auto prob_of = [&](int col) -> float {
            if (NPL > 0) {
                float v = 0.f;
#pragma unroll
                for (int k = 0; k < NR; k++) { float t = __shfl_sync(0xffffffffu, x[k], col & 31); if (k == (col >> 5)) v = t; }
                return v;
            }
            return row[col];
        };

        float weight = 1.0f, loss = 0.f;
        if (endpoint_path) {
            const int start = c_start, end = c_end;
            if (start != end) {
                if (NPL > 0) {                       // sparse lookups go through shared memory
#pragma unroll
                    for (int k = 0; k < NR; k++) if (lane + 32 * k < V) row[lane + 32 * k] = x[k];
                    __syncwarp();
                }
                int total = 0;
                for (int e = start + lane; e < end; e += 32) total += counts_val[e];
                total = warp_sum_i(total);
                const float total_f = (float)total;
                if (mode == 0) {
                    if (entropy_lambda > 0.0f && (end - start) > 1) {
                        float Hh = 0.f;
                        for (int e = start + lane; e < end; e += 32) {
                            float qe = counts_val[e] / total_f;
                            if (qe > 0.f) Hh -= qe * logf(qe);
                        }
                        Hh = warp_sum(Hh);
                        weight = 1.0f + entropy_lambda * (Hh / logf((float)V));
                    }
                    if (mass_weights) weight *= mass_w;
                }
                for (int e = start + lane; e < end; e += 32) {
                    int tok = counts_tok[e];
                    if ((unsigned)tok >= (unsigned)V) continue;      // a token outside the vocabulary is ignored, not written
                    float tgt = counts_val[e] / total_f;
                    float pr = row[tok];
                    loss -= tgt * logf(pr + 1e-10f);
                    row[tok] = pr - tgt;                             // tokens of one node are distinct
                }
                loss = warp_sum(loss) * weight;
                __syncwarp();
                if (NPL > 0) {
#pragma unroll
                    for (int k = 0; k < NR; k++) if (lane + 32 * k < V) x[k] = row[lane + 32 * k];
                }
            }
            // else: no observed continuation -- zero loss, and the row keeps the plain probabilities
        } else {
            if ((unsigned)target >= (unsigned)V) target = 0;         // never index outside the row
            weight = intermediate_weight;
            if (mass_weights) weight *= mass_w;
            const float pr = prob_of(target);
            loss = -logf(pr + 1e-10f) * weight;
            if (NPL > 0) {
#pragma unroll
                for (int k = 0; k < NR; k++) if (lane + 32 * k == target) x[k] -= 1.0f;
            } else {
                __syncwarp();
                if (lane == 0) row[target] = pr - 1.0f;
            }
        }
        if (NPL > 0) {
#pragma unroll
            for (int k = 0; k < NR; k++) if (lane + 32 * k < V) __stcs(g + lane + 32 * k, x[k] * weight);
            __syncwarp();                            // the next row may reuse the shared row
        } else {
            __syncwarp();
            for (int j = lane; j < V; j += 32) __stcs(g + j, row[j] * weight);
            __syncwarp();
        }
        if (lane == 0) loss_out[qi] = loss;
    }
}

// ---- batch form of the loss (V <= 256): one warp per 32 consecutive rows, one lane per row ------------------------
// The 32 rows of a batch are contiguous in memory (32*V floats, a multiple of 128 bytes), so the warp brings them
// into shared memory with ONE bulk asynchronous copy (cp.async.bulk, completion on an mbarrier) and writes the
// gradient rows back with one bulk store: full-line traffic although single rows (260 bytes at V = 65) straddle
// sectors, and the whole batch is in flight at once.  While the copy runs, lane l walks the dependent index chain
// of row l.  Then lane l owns row l: maximum, exponentials and sum, scaling -- three sweeps over its row in shared
// memory (column order skewed by the lane when V is even, so that the 32 lanes hit 32 banks), no shuffles.  The
// sparse count entries of an endpoint row are applied by its lane.  The wait on the mbarrier is bounded: if it ran
// out the warp sets bit 0 of the device status word and returns without storing.
__device__ int g_device_status = 0;

// 2^x for x <= 0 (softmax exponents): the hardware approximation, relative error about 2^-22; flushes below 2^-126
__device__ __forceinline__ float fast_exp2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

#define LOSSB_WARPS 4
#define LOSSB_WAIT_LIMIT (1 << 22)
__global__ void __launch_bounds__(LOSSB_WARPS * 32)
loss_batch_kernel(const float *__restrict__ logits, const int32_t *__restrict__ query_to_node,
                  const int32_t *__restrict__ query_offsets, const int32_t *__restrict__ ids,
                  const int32_t *__restrict__ token_ids, const int32_t *__restrict__ counts_offset,
                  const int32_t *__restrict__ counts_tok, const int32_t *__restrict__ counts_val,
                  const float *__restrict__ mass_weights, float *__restrict__ d_logits, float *__restrict__ loss_out,
                  int64_t T_q, int V, float entropy_lambda, float intermediate_weight, int ce_only, int mode, int aligned16) {
    extern __shared__ __align__(128) unsigned char lossb_smem[];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int64_t r0 = ((int64_t)blockIdx.x * LOSSB_WARPS + warp) * 32;
    if (r0 >= T_q) return;                                  // whole warp; warps of a block never synchronise with each other
    const int nrows = (T_q - r0 < 32) ? (int)(T_q - r0) : 32;
    float *tile = reinterpret_cast<float *>(lossb_smem) + (size_t)warp * 32 * V;
    uint64_t *bar = reinterpret_cast<uint64_t *>(lossb_smem + (size_t)LOSSB_WARPS * 32 * V * sizeof(float)) + warp;
    const uint32_t bytes = (uint32_t)nrows * V * sizeof(float);
    const bool bulk = aligned16 && (bytes & 15u) == 0;
    const float *src = logits + r0 * V;
    float *dst = d_logits + r0 * V;
    if (bulk) {
        if (lane == 0) {
            asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_u32(bar)));
            asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
            asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
            asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(smem_u32(tile)),
                         "l"(src), "r"(bytes), "r"(smem_u32(bar))
                         : "memory");
        }
    } else {
        for (int i = lane; i < nrows * V; i += 32) tile[i] = __ldcs(src + i);
    }

    // the row's index chain (query -> node -> offsets), 32 chains in flight per warp
    bool endpoint_path = false;
    int target = 0, c_start = 0, c_end = 0;
    float mass_w = 1.0f;
    const int64_t qi = r0 + lane;
    if (lane < nrows) {
        int cid = 0;
        if (mode == 1) { endpoint_path = true; cid = ids[qi]; }
        else {
            int n_idx = query_to_node[qi];
            bool is_endpoint = (qi + 1) == query_offsets[n_idx + 1];
            bool ce_as_intermediate = ce_only && is_endpoint && (qi + 1 < T_q);
            endpoint_path = is_endpoint && !ce_as_intermediate;
            if (endpoint_path) cid = ids[n_idx];
        }
        if (endpoint_path) { c_start = counts_offset[cid]; c_end = counts_offset[cid + 1]; }
        else target = token_ids[qi + 1];
        if (mode == 0 && mass_weights) mass_w = mass_weights[qi];
    }
    // an endpoint row's first count entries are fetched now, under the bulk copy, instead of as three dependent
    // global-memory loops after it (nearly every batch holds an endpoint row, and its lane would stall the warp)
    constexpr int CPRE = 8;
    int ptok[CPRE], pval[CPRE];
    const int ncnt = c_end - c_start;
#pragma unroll
    for (int e = 0; e < CPRE; e++) {
        ptok[e] = e < ncnt ? counts_tok[c_start + e] : -1;
        pval[e] = e < ncnt ? counts_val[c_start + e] : 0;
    }

    if (bulk) {
        uint32_t done = 0;
        if (lane == 0) {
            for (int it = 0; it < LOSSB_WAIT_LIMIT && !done; it++)
                asm volatile("{ .reg .pred p; mbarrier.try_wait.parity.shared::cta.b64 p, [%1], 0; selp.u32 %0, 1, 0, p; }"
                             : "=r"(done)
                             : "r"(smem_u32(bar))
                             : "memory");
            if (!done) atomicOr(&g_device_status, 1);
        }
        done = __shfl_sync(0xffffffffu, done, 0);
        if (!done) return;
    } else {
        __syncwarp();
    }

    float loss = 0.f;
    if (lane < nrows) {
        float *row = tile + lane * V;
        // lane-skewed column order: with row stride V the banks of the 32 lanes differ iff the per-lane step V + skew
        // is odd, so an even V starts lane l at column l (two plain segments: [first, V) then [0, first)).  When V is a
        // multiple of 4 the row is swept in 16-byte pieces instead (a quarter of the shared-memory instructions); there
        // eight neighbouring lanes must fall into different 16-byte bank groups, which a V that is a multiple of 8
        // needs a skew of one piece per lane for.
        const bool vec = (V & 3) == 0;
        const int V4 = V >> 2;
        const int first = vec ? ((V & 7) ? 0 : (lane % V4)) : ((V & 1) ? 0 : (lane % V));
        float4 *row4 = reinterpret_cast<float4 *>(row);
        float mx = -3.402823466e+38f;
        if (vec) {
            float m0 = mx, m1 = mx, m2 = mx, m3 = mx;
            for (int jj = 0; jj < V4; jj++) {
                int j = first + jj; if (j >= V4) j -= V4;
                const float4 x = row4[j];
                m0 = fmaxf(m0, x.x); m1 = fmaxf(m1, x.y); m2 = fmaxf(m2, x.z); m3 = fmaxf(m3, x.w);
            }
            mx = fmaxf(fmaxf(m0, m1), fmaxf(m2, m3));
        } else {
            float m0 = mx, m1 = mx, m2 = mx, m3 = mx;
            int j = first;
            for (; j + 3 < V; j += 4) { m0 = fmaxf(m0, row[j]); m1 = fmaxf(m1, row[j + 1]); m2 = fmaxf(m2, row[j + 2]); m3 = fmaxf(m3, row[j + 3]); }
            for (; j < V; j++) m0 = fmaxf(m0, row[j]);
            for (j = 0; j < first; j++) m1 = fmaxf(m1, row[j]);
            mx = fmaxf(fmaxf(m0, m1), fmaxf(m2, m3));
        }
        float sum = 0.f;
        const float mxl = mx * LOG2E;
        if (vec) {
            float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
            for (int jj = 0; jj < V4; jj++) {
                int j = first + jj; if (j >= V4) j -= V4;
                float4 x = row4[j];
                x.x = fast_exp2(fmaf(x.x, LOG2E, -mxl)); x.y = fast_exp2(fmaf(x.y, LOG2E, -mxl));
                x.z = fast_exp2(fmaf(x.z, LOG2E, -mxl)); x.w = fast_exp2(fmaf(x.w, LOG2E, -mxl));
                row4[j] = x;
                s0 += x.x; s1 += x.y; s2 += x.z; s3 += x.w;
            }
            sum = (s0 + s1) + (s2 + s3);
        } else {
            float s0 = 0.f, s1 = 0.f, s2 = 0.f, s3 = 0.f;
            int j = first;
            for (; j + 3 < V; j += 4) {
                const float e0 = fast_exp2(fmaf(row[j], LOG2E, -mxl)), e1 = fast_exp2(fmaf(row[j + 1], LOG2E, -mxl));
                const float e2 = fast_exp2(fmaf(row[j + 2], LOG2E, -mxl)), e3 = fast_exp2(fmaf(row[j + 3], LOG2E, -mxl));
                row[j] = e0; row[j + 1] = e1; row[j + 2] = e2; row[j + 3] = e3;
                s0 += e0; s1 += e1; s2 += e2; s3 += e3;
            }
            for (; j < V; j++) { const float e = fast_exp2(fmaf(row[j], LOG2E, -mxl)); row[j] = e; s0 += e; }
            for (j = 0; j < first; j++) { const float e = fast_exp2(fmaf(row[j], LOG2E, -mxl)); row[j] = e; s1 += e; }
            sum = (s0 + s1) + (s2 + s3);
        }
        const float inv = 1.0f / sum;
        float weight = 1.0f, total_f = 1.0f;
        if (endpoint_path) {
            if (c_start != c_end) {
                int total = 0;
#pragma unroll
                for (int e = 0; e < CPRE; e++) total += pval[e];
                for (int e = c_start + CPRE; e < c_end; e++) total += counts_val[e];
                total_f = (float)total;
                if (mode == 0) {
                    if (entropy_lambda > 0.0f && ncnt > 1) {
                        float Hh = 0.f;
#pragma unroll
                        for (int e = 0; e < CPRE; e++) {
                            float qe = pval[e] / total_f;
                            if (e < ncnt && qe > 0.f) Hh -= qe * logf(qe);
                        }
                        for (int e = c_start + CPRE; e < c_end; e++) {
                            float qe = counts_val[e] / total_f;
                            if (qe > 0.f) Hh -= qe * logf(qe);
                        }
                        weight = 1.0f + entropy_lambda * (Hh / logf((float)V));
                    }
                    if (mass_weights) weight *= mass_w;
                }
#pragma unroll
                for (int e = 0; e < CPRE; e++)                       // a token outside the vocabulary is ignored, not written
                    if ((unsigned)ptok[e] < (unsigned)V) loss -= (pval[e] / total_f) * logf(row[ptok[e]] * inv + 1e-10f);
                for (int e = c_start + CPRE; e < c_end; e++) {
                    int tok = counts_tok[e];
                    if ((unsigned)tok >= (unsigned)V) continue;
                    loss -= (counts_val[e] / total_f) * logf(row[tok] * inv + 1e-10f);
                }
                loss *= weight;
            }
            // else: no observed continuation -- zero loss, and the row keeps the plain probabilities
        } else {
            if ((unsigned)target >= (unsigned)V) target = 0;         // never index outside the row
            weight = intermediate_weight;
            if (mass_weights) weight *= mass_w;
            loss = -logf(row[target] * inv + 1e-10f) * weight;
        }
        const float f = inv * weight;
        if (vec) {
            for (int jj = 0; jj < V4; jj++) {
                int j = first + jj; if (j >= V4) j -= V4;
                float4 x = row4[j];
                x.x *= f; x.y *= f; x.z *= f; x.w *= f;
                row4[j] = x;
            }
        } else {
            int j = first;
            for (; j + 3 < V; j += 4) { row[j] *= f; row[j + 1] *= f; row[j + 2] *= f; row[j + 3] *= f; }
            for (; j < V; j++) row[j] *= f;
            for (j = 0; j < first; j++) row[j] *= f;
        }
        if (endpoint_path) {
#pragma unroll
            for (int e = 0; e < CPRE; e++)                           // tokens of one node are distinct
                if ((unsigned)ptok[e] < (unsigned)V) row[ptok[e]] -= (pval[e] / total_f) * weight;
            for (int e = c_start + CPRE; e < c_end; e++) {
                int tok = counts_tok[e];
                if ((unsigned)tok < (unsigned)V) row[tok] -= (counts_val[e] / total_f) * weight;
            }
        } else {
            row[target] -= weight;
        }
        loss_out[qi] = loss;
    }
    if (bulk) {
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");     // the rows written above become visible to the bulk store
        __syncwarp();
        if (lane == 0) {
            asm volatile("cp.async.bulk.global.shared::cta.bulk_group [%0], [%1], %2;" ::"l"(dst), "r"(smem_u32(tile)), "r"(bytes) : "memory");
            asm volatile("cp.async.bulk.commit_group;" ::: "memory");
            asm volatile("cp.async.bulk.wait_group.read 0;" ::: "memory");   // shared memory must outlive the read
        }
    } else {
        __syncwarp();
        for (int i = lane; i < nrows * V; i += 32) __stcs(dst + i, tile[i]);
    }
}

template <typename... Args>
static int launch_loss(int64_t rows, int V, cudaStream_t st, const float *logits, float *dlogits, Args... args) {
    if (V <= 256) {
        const size_t smem = (size_t)LOSSB_WARPS * 32 * V * sizeof(float) + LOSSB_WARPS * sizeof(uint64_t);
        static bool attr_set[64];
        int dev = 0;
        cudaGetDevice(&dev);
        if (dev >= 0 && dev < 64 && !attr_set[dev]) {
            CUDA_TRY(cudaFuncSetAttribute(loss_batch_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, LOSSB_WARPS * 32 * 256 * 4 + 64));
            attr_set[dev] = true;
        }
        const int rows_per_block = LOSSB_WARPS * 32;
        const unsigned blocks = (unsigned)((rows + rows_per_block - 1) / rows_per_block);
        const int aligned16 = ((reinterpret_cast<uintptr_t>(logits) | reinterpret_cast<uintptr_t>(dlogits)) & 15) == 0;
        loss_batch_kernel<<<blocks, LOSSB_WARPS * 32, smem, st>>>(args..., aligned16);
        return AGPT_OK;
    }
    const unsigned blocks = (unsigned)((rows + LOSS_ROWS_PER_BLOCK - 1) / LOSS_ROWS_PER_BLOCK);
    const size_t smem = (size_t)LOSS_WPB * V * sizeof(float);
    loss_kernel<0><<<blocks, LOSS_WPB * 32, smem, st>>>(args...);
    return AGPT_OK;
}

extern "C" int agpt_b200_device_status(int32_t *status_out) {
    if (!status_out) return agpt_set_error(AGPT_E_ARG, "device_status: null output");
    int v = 0;
    CUDA_TRY(cudaMemcpyFromSymbol(&v, g_device_status, sizeof(int)));      // synchronises with the work issued so far
    *status_out = v;
    return AGPT_OK;
}

extern "C" int agpt_b200_loss_per_query(const float *d_logits, const int32_t *d_query_to_node, const int32_t *d_query_offsets,
                                        const int32_t *d_radix_ids, const int32_t *d_token_ids, const int32_t *d_counts_offset,
                                        const int32_t *d_counts_tok, const int32_t *d_counts_val, const float *d_mass_weights,
                                        float *d_dlogits, float *d_loss, int64_t T_q, int V, float entropy_lambda,
                                        float intermediate_weight, int ce_only, void *stream) {
    if (!d_logits || !d_query_to_node || !d_query_offsets || !d_radix_ids || !d_token_ids || !d_counts_offset || !d_counts_tok ||
        !d_counts_val || !d_dlogits || !d_loss || T_q < 0 || V < 1)
        return agpt_set_error(AGPT_E_ARG, "loss_per_query: bad argument");
    if (T_q == 0) return AGPT_OK;
    if (V > 1400) return agpt_set_error(AGPT_E_LIMIT, "loss_per_query: vocabulary %d beyond 1400", V);
    int rc = launch_loss(T_q, V, (cudaStream_t)stream, d_logits, d_dlogits, d_logits, d_query_to_node, d_query_offsets, d_radix_ids, d_token_ids, d_counts_offset,
                d_counts_tok, d_counts_val, d_mass_weights, d_dlogits, d_loss, T_q, V, entropy_lambda, intermediate_weight, ce_only, 0);
    if (rc) return rc;
    return launch_status("loss_per_query");
}

extern "C" int agpt_b200_loss_per_node(const float *d_logits, const int32_t *d_node_ids, const int32_t *d_counts_offset,
                                       const int32_t *d_counts_tok, const int32_t *d_counts_val, float *d_dlogits, float *d_loss,
                                       int64_t N, int V, void *stream) {
    if (!d_logits || !d_node_ids || !d_counts_offset || !d_counts_tok || !d_counts_val || !d_dlogits || !d_loss || N < 0 || V < 1)
        return agpt_set_error(AGPT_E_ARG, "loss_per_node: bad argument");
    if (N == 0) return AGPT_OK;
    if (V > 1400) return agpt_set_error(AGPT_E_LIMIT, "loss_per_node: vocabulary %d beyond 1400", V);
    int rc = launch_loss(N, V, (cudaStream_t)stream, d_logits, d_dlogits, d_logits, (const int32_t *)nullptr, (const int32_t *)nullptr, d_node_ids,
                (const int32_t *)nullptr, d_counts_offset, d_counts_tok, d_counts_val, (const float *)nullptr, d_dlogits, d_loss, N, V,
                0.f, 1.f, 0, 1);
    if (rc) return rc;
    return launch_status("loss_per_node");
}

// --------------------------------------------------------------------------------------
// legacy packed-prefix kernels: one warp per (query, head), lanes over packed rows
// --------------------------------------------------------------------------------------
__device__ __forceinline__ void packed_query_span(const int *query_to_node, const int *query_offsets, const int *kv_offsets,
                                                  const int *kv_lengths, int t, int &node, int &len, int64_t &off) {
    node = query_to_node ? query_to_node[t] : t;
    len = query_to_node ? kv_lengths[node] - (query_offsets[node + 1] - t) + 1 : kv_lengths[node];
    off = kv_offsets[node];
}

template <int HD>
__global__ void packed_fwd_kernel(const float *__restrict__ q, const float *__restrict__ k, const float *__restrict__ v,
                                  const int *__restrict__ query_to_node, const int *__restrict__ query_offsets,
                                  const int *__restrict__ kv_offsets, const int *__restrict__ kv_lengths,
                                  float *__restrict__ out, float *__restrict__ weights, int T_q, int H, int max_len, float scale) {
    int64_t wid = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (wid >= (int64_t)T_q * H) return;
    const int lane = threadIdx.x & 31;
    const int t = (int)(wid / H), h = (int)(wid % H);
    int node, len;
    int64_t off;
    packed_query_span(query_to_node, query_offsets, kv_offsets, kv_lengths, t, node, len, off);
    float qv[HD];
#pragma unroll
    for (int c = 0; c < HD / 4; c++) {
        float4 x = ld4(q + ((int64_t)t * H + h) * HD + c * 4);
        qv[4 * c] = x.x; qv[4 * c + 1] = x.y; qv[4 * c + 2] = x.z; qv[4 * c + 3] = x.w;
    }
    float *wr = weights + ((int64_t)t * H + h) * max_len;
    float mx = -INFINITY;
    for (int p = lane; p < len; p += 32) {
        const float *kr = k + ((off + p) * H + h) * HD;
        float d = 0.f;
#pragma unroll
        for (int c = 0; c < HD / 4; c++) {
            float4 kk = ld4(kr + c * 4);
            d = fmaf(qv[4 * c], kk.x, d); d = fmaf(qv[4 * c + 1], kk.y, d);
            d = fmaf(qv[4 * c + 2], kk.z, d); d = fmaf(qv[4 * c + 3], kk.w, d);
        }
        d *= scale;
        wr[p] = d;
        mx = fmaxf(mx, d);
    }
    mx = warp_max(mx);
    float sum = 0.f;
    for (int p = lane; p < len; p += 32) { float e = expf(wr[p] - mx); wr[p] = e; sum += e; }
    sum = warp_sum(sum);
    const float inv = 1.0f / sum;
    float acc[HD];
#pragma unroll
    for (int d = 0; d < HD; d++) acc[d] = 0.f;
    for (int p = lane; p < max_len; p += 32) {
        if (p >= len) { wr[p] = 0.f; continue; }
        float w = wr[p] * inv;
        wr[p] = w;
        const float *vr = v + ((off + p) * H + h) * HD;
#pragma unroll
        for (int c = 0; c < HD / 4; c++) {
            float4 vv = ld4(vr + c * 4);
            acc[4 * c] = fmaf(w, vv.x, acc[4 * c]); acc[4 * c + 1] = fmaf(w, vv.y, acc[4 * c + 1]);
            acc[4 * c + 2] = fmaf(w, vv.z, acc[4 * c + 2]); acc[4 * c + 3] = fmaf(w, vv.w, acc[4 * c + 3]);
        }
    }
#pragma unroll
    for (int d = 0; d < HD; d++) acc[d] = warp_sum(acc[d]);
    if (lane == 0) {
        float *o = out + ((int64_t)t * H + h) * HD;
#pragma unroll
        for (int c = 0; c < HD / 4; c++) *reinterpret_cast<float4 *>(o + c * 4) = make_float4(acc[4 * c], acc[4 * c + 1], acc[4 * c + 2], acc[4 * c + 3]);
    }
}

// One warp per (node, head); the node's queries are visited in order and lane p%32 owns packed row p, so
// every dk_full/dv_full element is accumulated by one lane in a fixed order.
template <int HD>
__global__ void packed_bwd_kernel(const float *__restrict__ q, const float *__restrict__ k, const float *__restrict__ v,
                                  const float *__restrict__ weights, const float *__restrict__ d_out,
                                  const int *__restrict__ query_offsets, const int *__restrict__ kv_offsets,
                                  const int *__restrict__ kv_lengths, float *__restrict__ dq, float *__restrict__ dk_full,
                                  float *__restrict__ dv_full, int n_nodes, int H, int max_len, float scale, int accumulate) {
    int64_t wid = (int64_t)blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (wid >= (int64_t)n_nodes * H) return;
    const int lane = threadIdx.x & 31;
    const int node = (int)(wid / H), h = (int)(wid % H);
    const int q0 = query_offsets ? query_offsets[node] : node;
    const int q1 = query_offsets ? query_offsets[node + 1] : node + 1;
    const int klen = kv_lengths[node];
    const int64_t off = kv_offsets[node];
    for (int t = q0; t < q1; t++) {
        const int len = klen - (q1 - t) + 1;
        float qv[HD], gv[HD], dqa[HD];
#pragma unroll
        for (int c = 0; c < HD / 4; c++) {
            float4 x = ld4(q + ((int64_t)t * H + h) * HD + c * 4), y = ld4(d_out + ((int64_t)t * H + h) * HD + c * 4);
            qv[4 * c] = x.x; qv[4 * c + 1] = x.y; qv[4 * c + 2] = x.z; qv[4 * c + 3] = x.w;
            gv[4 * c] = y.x; gv[4 * c + 1] = y.y; gv[4 * c + 2] = y.z; gv[4 * c + 3] = y.w;
            dqa[4 * c] = dqa[4 * c + 1] = dqa[4 * c + 2] = dqa[4 * c + 3] = 0.f;
        }
        const float *wr = weights + ((int64_t)t * H + h) * max_len;
        float dot = 0.f;
        for (int p = lane; p < len; p += 32) {
            const float *vr = v + ((off + p) * H + h) * HD;
            float d = 0.f;
#pragma unroll
            for (int c = 0; c < HD / 4; c++) {
                float4 vv = ld4(vr + c * 4);
                d = fmaf(gv[4 * c], vv.x, d); d = fmaf(gv[4 * c + 1], vv.y, d);
                d = fmaf(gv[4 * c + 2], vv.z, d); d = fmaf(gv[4 * c + 3], vv.w, d);
            }
            dot = fmaf(d, wr[p], dot);
        }
        dot = warp_sum(dot);
        for (int p = lane; p < len; p += 32) {
            const float *kr = k + ((off + p) * H + h) * HD;
            const float *vr = v + ((off + p) * H + h) * HD;
            float *dkr = dk_full + ((off + p) * H + h) * HD, *dvr = dv_full + ((off + p) * H + h) * HD;
            const float w = wr[p];
            float d = 0.f;
#pragma unroll
            for (int c = 0; c < HD / 4; c++) {
                float4 vv = ld4(vr + c * 4);
                d = fmaf(gv[4 * c], vv.x, d); d = fmaf(gv[4 * c + 1], vv.y, d);
                d = fmaf(gv[4 * c + 2], vv.z, d); d = fmaf(gv[4 * c + 3], vv.w, d);
            }
            const float ds = w * (d - dot) * scale;
            const bool add = accumulate || t > q0;
#pragma unroll
            for (int c = 0; c < HD / 4; c++) {
                float4 kk = ld4(kr + c * 4);
                dqa[4 * c] = fmaf(ds, kk.x, dqa[4 * c]); dqa[4 * c + 1] = fmaf(ds, kk.y, dqa[4 * c + 1]);
                dqa[4 * c + 2] = fmaf(ds, kk.z, dqa[4 * c + 2]); dqa[4 * c + 3] = fmaf(ds, kk.w, dqa[4 * c + 3]);
                float4 a = make_float4(0.f, 0.f, 0.f, 0.f), b = a;
                if (add) { a = *reinterpret_cast<float4 *>(dkr + c * 4); b = *reinterpret_cast<float4 *>(dvr + c * 4); }
                a.x = fmaf(ds, qv[4 * c], a.x); a.y = fmaf(ds, qv[4 * c + 1], a.y); a.z = fmaf(ds, qv[4 * c + 2], a.z); a.w = fmaf(ds, qv[4 * c + 3], a.w);
                b.x = fmaf(w, gv[4 * c], b.x); b.y = fmaf(w, gv[4 * c + 1], b.y); b.z = fmaf(w, gv[4 * c + 2], b.z); b.w = fmaf(w, gv[4 * c + 3], b.w);
                *reinterpret_cast<float4 *>(dkr + c * 4) = a;
                *reinterpret_cast<float4 *>(dvr + c * 4) = b;
            }
        }
#pragma unroll
        for (int d = 0; d < HD; d++) dqa[d] = warp_sum(dqa[d]);
        if (lane == 0) {
            float *o = dq + ((int64_t)t * H + h) * HD;
#pragma unroll
            for (int c = 0; c < HD / 4; c++) *reinterpret_cast<float4 *>(o + c * 4) = make_float4(dqa[4 * c], dqa[4 * c + 1], dqa[4 * c + 2], dqa[4 * c + 3]);
        }
        __syncwarp();
    }
}

static void legacy_fwd(const float *q, const float *k, const float *v, const int *q2n, const int *qoff, const int *kvo,
                       const int *kvl, float *out, float *w, int T_q, int H, int hd, int max_len, float scale) {
    if (T_q <= 0) return;
    const int wpb = 4;
    unsigned blocks = (unsigned)(((int64_t)T_q * H + wpb - 1) / wpb);
    switch (hd) {
        case 16: packed_fwd_kernel<16><<<blocks, wpb * 32>>>(q, k, v, q2n, qoff, kvo, kvl, out, w, T_q, H, max_len, scale); break;
        case 32: packed_fwd_kernel<32><<<blocks, wpb * 32>>>(q, k, v, q2n, qoff, kvo, kvl, out, w, T_q, H, max_len, scale); break;
        case 64: packed_fwd_kernel<64><<<blocks, wpb * 32>>>(q, k, v, q2n, qoff, kvo, kvl, out, w, T_q, H, max_len, scale); break;
        default: agpt_set_error(AGPT_E_ARG, "legacy attention: head_dim %d unsupported (16, 32 or 64)", hd); return;
    }
    launch_status("legacy attention forward");
}

static void legacy_bwd(const float *q, const float *k, const float *v, const float *w, const float *d_out, const int *qoff,
                       const int *kvo, const int *kvl, float *dq, float *dk, float *dv, int n_nodes, int H, int hd, int max_len,
                       float scale, int accumulate) {
    if (n_nodes <= 0) return;
    const int wpb = 4;
    unsigned blocks = (unsigned)(((int64_t)n_nodes * H + wpb - 1) / wpb);
    switch (hd) {
        case 16: packed_bwd_kernel<16><<<blocks, wpb * 32>>>(q, k, v, w, d_out, qoff, kvo, kvl, dq, dk, dv, n_nodes, H, max_len, scale, accumulate); break;
        case 32: packed_bwd_kernel<32><<<blocks, wpb * 32>>>(q, k, v, w, d_out, qoff, kvo, kvl, dq, dk, dv, n_nodes, H, max_len, scale, accumulate); break;
        case 64: packed_bwd_kernel<64><<<blocks, wpb * 32>>>(q, k, v, w, d_out, qoff, kvo, kvl, dq, dk, dv, n_nodes, H, max_len, scale, accumulate); break;
        default: agpt_set_error(AGPT_E_ARG, "legacy attention backward: head_dim %d unsupported (16, 32 or 64)", hd); return;
    }
    launch_status("legacy attention backward");
}

extern "C" void cuda_batched_varlen_attention(const float *q, const float *k, const float *v, const int *kv_offsets,
                                              const int *kv_lengths, float *output, float *weights_out, int n_nodes, int n_heads,
                                              int head_dim, int max_len, float scale) {
    legacy_fwd(q, k, v, nullptr, nullptr, kv_offsets, kv_lengths, output, weights_out, n_nodes, n_heads, head_dim, max_len, scale);
}

extern "C" void cuda_batched_varlen_attention_backward(const float *q, const float *k, const float *v, const float *w,
                                                       const float *d_out, const int *kv_offsets, const int *kv_lengths, float *dq,
                                                       float *dk_full, float *dv_full, int n_nodes, int n_heads, int head_dim,
                                                       int max_len, float scale) {
    legacy_bwd(q, k, v, w, d_out, nullptr, kv_offsets, kv_lengths, dq, dk_full, dv_full, n_nodes, n_heads, head_dim, max_len, scale, 0);
}

extern "C" void cuda_batched_varlen_attention_L_queries(const float *q, const float *k, const float *v, const int *query_to_node,
                                                        const int *query_offsets, const int *kv_offsets, const int *kv_lengths,
                                                        float *output, float *weights_out, int T_q, int n_heads, int head_dim,
                                                        int max_kv_len, float scale) {
    legacy_fwd(q, k, v, query_to_node, query_offsets, kv_offsets, kv_lengths, output, weights_out, T_q, n_heads, head_dim, max_kv_len, scale);
}

// The node count is not an argument of the reference signature; it is query_to_node[T_q - 1] + 1.
extern "C" void cuda_batched_varlen_attention_L_queries_backward(const float *q, const float *k, const float *v, const float *w,
                                                                 const float *d_out, const int *query_to_node,
                                                                 const int *query_offsets, const int *kv_offsets,
                                                                 const int *kv_lengths, float *dq, float *dk_full, float *dv_full,
                                                                 int T_q, int n_heads, int head_dim, int max_kv_len, float scale) {
    if (T_q <= 0) return;
    int last = 0;
    if (cudaMemcpy(&last, query_to_node + (T_q - 1), sizeof(int), cudaMemcpyDeviceToHost) != cudaSuccess) {
        agpt_set_error(AGPT_E_CUDA, "L_queries_backward: cannot read query_to_node");
        return;
    }
    legacy_bwd(q, k, v, w, d_out, query_offsets, kv_offsets, kv_lengths, dq, dk_full, dv_full, last + 1, n_heads, head_dim, max_kv_len, scale, 1);
}

__global__ void copy_kernel(const float4 *__restrict__ src, float4 *__restrict__ dst, int64_t n4) {
    int64_t idx = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx < n4) dst[idx] = src[idx];
}
__global__ void copy_tail_kernel(const float *__restrict__ src, float *__restrict__ dst, int64_t from, int64_t n) {
    int64_t idx = from + (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx < n) dst[idx] = src[idx];
}

// [n*H, hd] and [n, H*hd] are the same bytes: a plain copy.
extern "C" void cuda_unpack_batched_attn_output(const float *packed_output, float *unpacked_output, int n_nodes, int n_heads, int head_dim) {
    int64_t total = (int64_t)n_nodes * n_heads * head_dim;
    if (total <= 0 || packed_output == unpacked_output) return;
    bool aligned = (((uintptr_t)packed_output | (uintptr_t)unpacked_output) & 15) == 0;
    int64_t n4 = aligned ? total / 4 : 0;
    if (n4) copy_kernel<<<(unsigned)((n4 + 255) / 256), 256>>>((const float4 *)packed_output, (float4 *)unpacked_output, n4);
    if (n4 * 4 < total) copy_tail_kernel<<<(unsigned)((total - n4 * 4 + 255) / 256), 256>>>(packed_output, unpacked_output, n4 * 4, total);
    launch_status("unpack");
}

extern "C" void cuda_sync(void) {
    cudaError_t e = cudaDeviceSynchronize();
    if (e != cudaSuccess) agpt_set_error(AGPT_E_CUDA, "cuda_sync: %s", cudaGetErrorString(e));
}

// --------------------------------------------------------------------------------------
// host-buffer step: upload, forward, backward and download as a three-stream pipeline over row chunks.
// Ancestors precede descendants in depth-first order, so once rows [0, e) are on the device every tile below e
// can run forward and backward: chunk c+1 uploads while chunk c computes and chunk c-1's out/lse/dq download.
// Only dK/dV (complete after the last tile and the reduction) download at the end.
// --------------------------------------------------------------------------------------
static int attn_fwd_bwd_host_impl(const agpt_plan *cp, const float *h_q, const float *h_k, const float *h_v,
                                  const float *h_dout, float *h_out, float *h_lse, float *h_dq, float *h_dk, float *h_dv,
                                  int kv_dtype, int n_heads, int head_dim, float scale);

extern "C" int agpt_b200_attn_fwd_bwd_host(const agpt_plan *cp, const float *h_q, const float *h_k, const float *h_v,
                                           const float *h_dout, float *h_out, float *h_lse, float *h_dq, float *h_dk, float *h_dv,
                                           int kv_dtype, int n_heads, int head_dim, float scale) {
    const int rc = attn_fwd_bwd_host_impl(cp, h_q, h_k, h_v, h_dout, h_out, h_lse, h_dq, h_dk, h_dv, kv_dtype, n_heads, head_dim, scale);
    if (rc != AGPT_OK && cp && cp->device >= 0) {
        // copies queued before the failure still read and write the caller's buffers (and the cached arena): wait for
        // them before the buffers go back to the caller
        for (void *st : cp->host_streams)
            if (st) cudaStreamSynchronize((cudaStream_t)st);
    }
    return rc;
}

static int attn_fwd_bwd_host_impl(const agpt_plan *cp, const float *h_q, const float *h_k, const float *h_v,
                                  const float *h_dout, float *h_out, float *h_lse, float *h_dq, float *h_dk, float *h_dv,
                                  int kv_dtype, int n_heads, int head_dim, float scale) {
    int rc = check_common(cp, n_heads, head_dim, "attn_fwd_bwd_host");
    if (rc) return rc;
    if (!h_q || !h_k || !h_v || !h_dout || !h_out || !h_lse || !h_dq || !h_dk || !h_dv)
        return agpt_set_error(AGPT_E_ARG, "attn_fwd_bwd_host: null buffer");
    if (kv_dtype != AGPT_KV_F32 && kv_dtype != AGPT_KV_BF16) return agpt_set_error(AGPT_E_ARG, "attn_fwd_bwd_host: bad kv_dtype");
    agpt_plan *p = const_cast<agpt_plan *>(cp);        // the cached arena is the only state a call changes
    CUDA_TRY(cudaSetDevice(p->device));
    const int D = n_heads * head_dim, M = p->tile_m;
    const int64_t n = p->n;
    const size_t rowb = (size_t)D * sizeof(float);
    const size_t tens = (((size_t)n * rowb) + 255) & ~(size_t)255;
    const size_t lseb = (((size_t)n * n_heads * sizeof(float)) + 255) & ~(size_t)255;
    const size_t wsb = (((size_t)agpt_b200_attn_bwd_workspace_bytes(p, D)) + 255) & ~(size_t)255;
    const bool bf = kv_dtype == AGPT_KV_BF16;
    // chunks of about 64 MB per tensor, whole tiles
    const int64_t ch_rows = std::max<int64_t>(M, ((64ll << 20) / (int64_t)rowb) / M * M);
    const int64_t n_ch = (n + ch_rows - 1) / ch_rows;
    const size_t fix_dev_cap = (((size_t)n_ch * (size_t)p->max_depth + p->multi_node.size()) * (2 * rowb + sizeof(int32_t)) + 511) & ~(size_t)255;
    const size_t need = 8 * tens + lseb + wsb + (bf ? tens : 0) + fix_dev_cap;
    if (p->host_arena_bytes < need) {
        if (p->host_arena) { CUDA_TRY(cudaFree(p->host_arena)); p->host_arena = nullptr; p->host_arena_bytes = 0; }
        CUDA_TRY(cudaMalloc(&p->host_arena, need));
        p->host_arena_bytes = need;
    }
    for (int i = 0; i < 3; i++)
        if (!p->host_streams[i]) { cudaStream_t st; CUDA_TRY(cudaStreamCreateWithFlags(&st, cudaStreamNonBlocking)); p->host_streams[i] = st; }
    cudaStream_t s_up = (cudaStream_t)p->host_streams[0], s_run = (cudaStream_t)p->host_streams[1], s_down = (cudaStream_t)p->host_streams[2];
    char *base = (char *)p->host_arena;
    float *dq_in = (float *)base, *dk_in = (float *)(base + tens), *dv_in = (float *)(base + 2 * tens), *dg = (float *)(base + 3 * tens);
    float *dout = (float *)(base + 4 * tens), *ddq = (float *)(base + 5 * tens), *ddk = (float *)(base + 6 * tens), *ddv = (float *)(base + 7 * tens);
    float *dlse = (float *)(base + 8 * tens);
    void *ws = base + 8 * tens + lseb;
    __nv_bfloat16 *kb = bf ? (__nv_bfloat16 *)(base + 8 * tens + lseb + wsb) : nullptr;
    __nv_bfloat16 *vb = bf ? kb + (size_t)n * D : nullptr;
    char *fix_dev = base + 8 * tens + lseb + wsb + (bf ? tens : 0);
    const void *kk = bf ? (const void *)kb : (const void *)dk_in, *vv = bf ? (const void *)vb : (const void *)dv_in;
    const int64_t rows = (int64_t)p->chain_ids.size();
    float *pk = (float *)ws, *pv = pk + rows * D, *segk = pv + rows * D, *segv = segk + p->n_multi_items * D;

    while ((int64_t)p->host_events.size() < 3 * n_ch + 1) {
        cudaEvent_t e;
        CUDA_TRY(cudaEventCreateWithFlags(&e, cudaEventDisableTiming));
        p->host_events.push_back(e);
    }
    auto ev = [&](int64_t c, int k) { return (cudaEvent_t)p->host_events[3 * c + k]; };
    // dK/dV rows of a chunk are final once every tile of their subtree has run and been reduced.  After chunk c
    // (rows below r1) that holds for all rows except the strict ancestors of row r1, whose subtrees go on, and
    // the few nodes whose reduction needs the second pass.  Chunks therefore download dK/dV right away and those
    // rows ("fix rows": at most depth per chunk boundary) are downloaded again at the end.
    std::vector<int32_t> fix(p->multi_node.begin(), p->multi_node.end());
    for (int64_t c = 0; c + 1 < n_ch; c++)
        for (int32_t a = p->parent_dfs[(c + 1) * ch_rows]; a >= 0; a = p->parent_dfs[a]) fix.push_back(a);
    std::sort(fix.begin(), fix.end());
    fix.erase(std::unique(fix.begin(), fix.end()), fix.end());
    const size_t nfix = fix.size();
    const size_t fix_bytes = nfix * (2 * rowb + sizeof(int32_t)) + 256;
    if (fix_dev_cap < fix_bytes) return agpt_set_error(AGPT_E_LIMIT, "attn_fwd_bwd_host: fix-row staging too small");
    if (p->host_fix_bytes < fix_bytes) {
        if (p->host_fix) { CUDA_TRY(cudaFreeHost(p->host_fix)); p->host_fix = nullptr; p->host_fix_bytes = 0; }
        CUDA_TRY(cudaMallocHost(&p->host_fix, fix_bytes));
        p->host_fix_bytes = fix_bytes;
    }
    int64_t item_done = 0;
    const int64_t n_items = (int64_t)p->item_node.size();
    for (int64_t c = 0; c < n_ch; c++) {
        const int64_t r0 = c * ch_rows, r1 = std::min(n, r0 + ch_rows), nr = r1 - r0;
        const size_t off = (size_t)r0 * D, bytes = (size_t)nr * rowb;
        CUDA_TRY(cudaMemcpyAsync(dq_in + off, h_q + off, bytes, cudaMemcpyHostToDevice, s_up));
        CUDA_TRY(cudaMemcpyAsync(dk_in + off, h_k + off, bytes, cudaMemcpyHostToDevice, s_up));
        CUDA_TRY(cudaMemcpyAsync(dv_in + off, h_v + off, bytes, cudaMemcpyHostToDevice, s_up));
        CUDA_TRY(cudaMemcpyAsync(dg + off, h_dout + off, bytes, cudaMemcpyHostToDevice, s_up));
        CUDA_TRY(cudaEventRecord(ev(c, 0), s_up));
        CUDA_TRY(cudaStreamWaitEvent(s_run, ev(c, 0), 0));
        if (bf) {
            if ((rc = agpt_b200_kv_store_write_bf16(dk_in + off, kb + off, nr, D, s_run))) return rc;
            if ((rc = agpt_b200_kv_store_write_bf16(dv_in + off, vb + off, nr, D, s_run))) return rc;
        }
        const int t0 = (int)(r0 / M), nt = (int)((r1 + M - 1) / M) - t0;
        if ((rc = fwd_dispatch(p, dq_in, kk, vv, kv_dtype, dout, dlse, n_heads, head_dim, scale, s_run, t0, nt))) return rc;
        CUDA_TRY(cudaEventRecord(ev(c, 1), s_run));
        if ((rc = bwd_dispatch(p, dq_in, kk, vv, kv_dtype, dout, dlse, dg, ddq, ddk, ddv, pk, pv, n_heads, head_dim, scale, s_run, t0, nt))) return rc;
        // every reduction item whose last tile has now run
        const int64_t item_end = std::upper_bound(p->item_t1.begin(), p->item_t1.end(), (int32_t)(t0 + nt - 1)) - p->item_t1.begin();
        if ((rc = run_reduce_range(p, pk, pv, segk, segv, ddk, ddv, D, s_run, item_done, item_end, c + 1 == n_ch))) return rc;
        item_done = item_end;
        CUDA_TRY(cudaEventRecord(ev(c, 2), s_run));
        CUDA_TRY(cudaStreamWaitEvent(s_down, ev(c, 1), 0));
        CUDA_TRY(cudaMemcpyAsync(h_out + off, dout + off, bytes, cudaMemcpyDeviceToHost, s_down));
        CUDA_TRY(cudaMemcpyAsync(h_lse + (size_t)r0 * n_heads, dlse + (size_t)r0 * n_heads, (size_t)nr * n_heads * sizeof(float), cudaMemcpyDeviceToHost, s_down));
        CUDA_TRY(cudaStreamWaitEvent(s_down, ev(c, 2), 0));
        CUDA_TRY(cudaMemcpyAsync(h_dq + off, ddq + off, bytes, cudaMemcpyDeviceToHost, s_down));
        CUDA_TRY(cudaMemcpyAsync(h_dk + off, ddk + off, bytes, cudaMemcpyDeviceToHost, s_down));
        CUDA_TRY(cudaMemcpyAsync(h_dv + off, ddv + off, bytes, cudaMemcpyDeviceToHost, s_down));
    }
    if (item_done != n_items) return agpt_set_error(AGPT_E_CUDA, "attn_fwd_bwd_host: reduction list not exhausted");
    if (nfix > 0) {
        // gather the fix rows (now final) and download them after the chunk downloads
        char *hf = (char *)p->host_fix;
        int32_t *h_idx = (int32_t *)(hf + nfix * 2 * rowb);
        std::copy(fix.begin(), fix.end(), h_idx);
        int32_t *d_idx = (int32_t *)(fix_dev + nfix * 2 * rowb);
        float *d_fk = (float *)fix_dev, *d_fv = d_fk + nfix * D;
        CUDA_TRY(cudaMemcpyAsync(d_idx, h_idx, nfix * sizeof(int32_t), cudaMemcpyHostToDevice, s_run));
        if ((rc = agpt_b200_gather_rows(ddk, d_idx, d_fk, (int64_t)nfix, D, s_run))) return rc;
        if ((rc = agpt_b200_gather_rows(ddv, d_idx, d_fv, (int64_t)nfix, D, s_run))) return rc;
        cudaEvent_t done = (cudaEvent_t)p->host_events[3 * n_ch];
        CUDA_TRY(cudaEventRecord(done, s_run));
        CUDA_TRY(cudaStreamWaitEvent(s_down, done, 0));
        CUDA_TRY(cudaMemcpyAsync(hf, d_fk, nfix * 2 * rowb, cudaMemcpyDeviceToHost, s_down));
    }
    CUDA_TRY(cudaStreamSynchronize(s_down));
    CUDA_TRY(cudaStreamSynchronize(s_run));
    CUDA_TRY(cudaStreamSynchronize(s_up));
    for (size_t i = 0; i < nfix; i++) {
        memcpy(h_dk + (size_t)fix[i] * D, (char *)p->host_fix + i * rowb, rowb);
        memcpy(h_dv + (size_t)fix[i] * D, (char *)p->host_fix + (nfix + i) * rowb, rowb);
    }
    return AGPT_OK;
}

// --------------------------------------------------------------------------------------
// backward without any allocation: scratch in a fixed device array
// --------------------------------------------------------------------------------------
// Some callers of this library cannot obtain device memory at the point where they run the backward
// pass: a host runtime that took the whole device at start-up and hands out slices of its own pool
// (so cudaMalloc would fail or fragment what is left), or a step whose buffer set was fixed once and
// must not grow.  For them the partial dK/dV rows live in this array instead of a caller workspace.
// It is part of the module image, so every GPU that loads the library holds AGPT_STATIC_SCRATCH_BYTES
// of it until the process exits.
#define AGPT_STATIC_SCRATCH_BYTES (64ll << 20)
static __device__ __align__(256) unsigned char g_static_scratch[AGPT_STATIC_SCRATCH_BYTES];

static void *g_static_scratch_addr[AGPT_MAX_DEVICES];   // device address of the array, per device; nullptr = not looked up yet

extern "C" int64_t agpt_b200_static_scratch_bytes(void) { return AGPT_STATIC_SCRATCH_BYTES; }

extern "C" int agpt_b200_attn_bwd_static(const agpt_plan *p, const float *d_q, const void *d_k, const void *d_v, int kv_dtype,
                                         const float *d_out, const float *d_lse, const float *d_dout, float *d_dq, float *d_dk,
                                         float *d_dv, int n_heads, int head_dim, float scale, void *stream) {
    int rc = check_common(p, n_heads, head_dim, "attn_bwd_static");
    if (rc) return rc;
    if (!d_q || !d_k || !d_v || !d_out || !d_lse || !d_dout || !d_dq || !d_dk || !d_dv)
        return agpt_set_error(AGPT_E_ARG, "attn_bwd_static: null buffer");
    if (kv_dtype != AGPT_KV_F32 && kv_dtype != AGPT_KV_BF16) return agpt_set_error(AGPT_E_ARG, "attn_bwd_static: bad kv_dtype");
    const int D = n_heads * head_dim;
    const int64_t need = agpt_b200_attn_bwd_workspace_bytes(p, D);
    if (need > AGPT_STATIC_SCRATCH_BYTES)
        return agpt_set_error(AGPT_E_LIMIT,
                              "attn_bwd_static: this plan needs %lld bytes of scratch, the built-in array holds %lld; "
                              "use agpt_b200_attn_bwd with a caller workspace or split the trie into smaller units",
                              (long long)need, (long long)AGPT_STATIC_SCRATCH_BYTES);
    int cur = -1;
    CUDA_TRY(cudaGetDevice(&cur));
    if (cur != p->device) return agpt_set_error(AGPT_E_ARG, "attn_bwd_static: current device %d is not the plan's device %d", cur, p->device);
    if (cur < 0 || cur >= AGPT_MAX_DEVICES) return agpt_set_error(AGPT_E_LIMIT, "attn_bwd_static: device index %d beyond %d", cur, AGPT_MAX_DEVICES);
    if (!g_static_scratch_addr[cur]) {
        // In host code the array's name is only a handle; the address a kernel can use comes from the runtime,
        // per device, with that device current.
        void *addr = nullptr;
        CUDA_TRY(cudaGetSymbolAddress(&addr, g_static_scratch));
        if (!addr) return agpt_set_error(AGPT_E_CUDA, "attn_bwd_static: cudaGetSymbolAddress returned a null address");
        g_static_scratch_addr[cur] = addr;
    }
    // Every partial row and every segment sum the reduction reads is written earlier in this same call, so nothing
    // left in the array by a previous call is ever read and nothing needs clearing.
    const int64_t rows = (int64_t)p->chain_ids.size();
    float *pk = (float *)g_static_scratch_addr[cur], *pv = pk + rows * D, *segk = pv + rows * D, *segv = segk + p->n_multi_items * D;
    rc = bwd_dispatch(p, d_q, d_k, d_v, kv_dtype, d_out, d_lse, d_dout, d_dq, d_dk, d_dv, pk, pv, n_heads, head_dim, scale,
                      (cudaStream_t)stream, 0, (int)p->n_tiles);
    if (rc) return rc;
    return run_reduce(p, pk, pv, segk, segv, d_dk, d_dv, D, (cudaStream_t)stream);
}
