// Suffix order of a token corpus on the GPU, for the radix-trie builder (trie_suffix.cpp).
//
// Start positions 0..n-2 are ordered by their first key_len tokens (a position past the end of the corpus orders
// before every token) with a least-significant-digit radix sort: one stable pass per token of the key, from the last
// token to the first.  Each pass is HBM-bound integer work: a gather of one token per suffix (the digit), then one
// 8- or 16-bit radix pass over (digit, position) pairs (cub::DeviceRadixSort, whose passes are stable).  Afterwards
// one thread per neighbouring pair counts the common leading tokens.  For the depth-32 trie of a 5M-token corpus
// this replaces about 80 s of bucket refinement on one host thread by a few milliseconds of device time; the
// linear-time assembly of the trie from the order stays on the host.
#include <cuda_runtime.h>

#include <cub/device/device_radix_sort.cuh>

#include <cstdint>

#include "../../include/agpt_b200.h"
#include "internal.h"

namespace {

#define CUDA_TRY(x)                                                                              \
    do {                                                                                         \
        cudaError_t e_ = (x);                                                                    \
        if (e_ != cudaSuccess) { rc = agpt_set_error(AGPT_E_CUDA, "%s: %s", #x, cudaGetErrorString(e_)); goto done; } \
    } while (0)

template <typename DT>
__global__ void __launch_bounds__(256) digit_kernel(const int32_t *__restrict__ corpus, const int32_t *__restrict__ sa, int64_t n, int32_t m,
                                                     int d, DT *__restrict__ digit) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < m; i += (int64_t)gridDim.x * blockDim.x) {
        const int64_t p = (int64_t)sa[i] + d;
        digit[i] = p < n ? (DT)(corpus[p] + 1) : (DT)0;
    }
}

__global__ void __launch_bounds__(256) iota_kernel(int32_t *__restrict__ sa, int32_t m) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < m; i += (int64_t)gridDim.x * blockDim.x) sa[i] = (int32_t)i;
}

// lcp[i] = number of equal leading tokens of the keys of sa[i-1] and sa[i] (tokens past the corpus end match nothing)
__global__ void __launch_bounds__(256) lcp_kernel(const int32_t *__restrict__ corpus, const int32_t *__restrict__ sa, int64_t n, int32_t m,
                                                   int key_len, int32_t *__restrict__ lcp) {
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < m; i += (int64_t)gridDim.x * blockDim.x) {
        if (i == 0) { lcp[0] = 0; continue; }
        const int64_t a = sa[i - 1], b = sa[i];
        int64_t lim = n - (a > b ? a : b);
        if (lim > key_len) lim = key_len;
        int l = 0;
        while (l < lim && corpus[a + l] == corpus[b + l]) l++;
        lcp[i] = l;
    }
}

template <typename DT>
int sort_suffixes(const int32_t *d_corpus, int64_t n, int32_t m, int key_len, int bits, int32_t *d_sa0, int32_t *d_sa1, int32_t **d_sorted,
                  cudaStream_t st) {
    int rc = AGPT_OK;
    DT *d_dig0 = nullptr, *d_dig1 = nullptr;
    void *d_tmp = nullptr;
    size_t tmp_bytes = 0;
    const unsigned grid = (unsigned)(((int64_t)m + 255) / 256 < 148 * 16 ? ((int64_t)m + 255) / 256 : 148 * 16);
    int32_t *in = d_sa0, *outp = d_sa1;
    CUDA_TRY(cudaMalloc(&d_dig0, (size_t)m * sizeof(DT)));
    CUDA_TRY(cudaMalloc(&d_dig1, (size_t)m * sizeof(DT)));
    CUDA_TRY(cub::DeviceRadixSort::SortPairs(nullptr, tmp_bytes, d_dig0, d_dig1, in, outp, m, 0, bits, st));
    CUDA_TRY(cudaMalloc(&d_tmp, tmp_bytes ? tmp_bytes : 16));
    iota_kernel<<<grid, 256, 0, st>>>(in, m);
    for (int d = key_len - 1; d >= 0; d--) {
        digit_kernel<DT><<<grid, 256, 0, st>>>(d_corpus, in, n, m, d, d_dig0);
        CUDA_TRY(cub::DeviceRadixSort::SortPairs(d_tmp, tmp_bytes, d_dig0, d_dig1, in, outp, m, 0, bits, st));
        int32_t *t = in; in = outp; outp = t;
    }
    CUDA_TRY(cudaGetLastError());
    *d_sorted = in;
done:
    cudaFree(d_dig0);
    cudaFree(d_dig1);
    cudaFree(d_tmp);
    return rc;
}

}  // namespace

extern "C" int agpt_b200_suffix_order_gpu(const int32_t *corpus, int64_t n, int key_len, int device, int32_t *sa_out, int32_t *lcp_out,
                                          float *device_ms_out) {
    if (!corpus || !sa_out || !lcp_out || n < 2 || key_len < 1) return agpt_set_error(AGPT_E_ARG, "suffix_order_gpu: bad argument");
    if (n >= (1LL << 31)) return agpt_set_error(AGPT_E_LIMIT, "suffix_order_gpu: corpus beyond 2^31 tokens");
    int vocab = 0;
    for (int64_t i = 0; i < n; i++) {
        if (corpus[i] < 0) return agpt_set_error(AGPT_E_ARG, "suffix_order_gpu: negative token");
        if (corpus[i] >= vocab) vocab = corpus[i] + 1;
    }
    if (vocab > 65534) return agpt_set_error(AGPT_E_LIMIT, "suffix_order_gpu: vocabulary beyond 65534");
    int rc = AGPT_OK;
    const int32_t m = (int32_t)(n - 1);
    int32_t *d_corpus = nullptr, *d_sa0 = nullptr, *d_sa1 = nullptr, *d_lcp = nullptr, *d_sorted = nullptr;
    cudaEvent_t e0 = nullptr, e1 = nullptr;
    cudaStream_t st = nullptr;
    int bits = 1;
    while ((1 << bits) < vocab + 1) bits++;
    CUDA_TRY(cudaSetDevice(device));
    CUDA_TRY(cudaStreamCreate(&st));
    CUDA_TRY(cudaEventCreate(&e0));
    CUDA_TRY(cudaEventCreate(&e1));
    CUDA_TRY(cudaMalloc(&d_corpus, (size_t)n * 4));
    CUDA_TRY(cudaMalloc(&d_sa0, (size_t)m * 4));
    CUDA_TRY(cudaMalloc(&d_sa1, (size_t)m * 4));
    CUDA_TRY(cudaMalloc(&d_lcp, (size_t)m * 4));
    CUDA_TRY(cudaMemcpyAsync(d_corpus, corpus, (size_t)n * 4, cudaMemcpyHostToDevice, st));
    CUDA_TRY(cudaEventRecord(e0, st));
    rc = vocab + 1 <= 256 ? sort_suffixes<uint8_t>(d_corpus, n, m, key_len, bits, d_sa0, d_sa1, &d_sorted, st)
                          : sort_suffixes<uint16_t>(d_corpus, n, m, key_len, bits, d_sa0, d_sa1, &d_sorted, st);
    if (rc) goto done;
    {
        const int64_t blocks = ((int64_t)m + 255) / 256;
        lcp_kernel<<<(unsigned)(blocks < 148 * 16 ? blocks : 148 * 16), 256, 0, st>>>(d_corpus, d_sorted, n, m, key_len, d_lcp);
    }
    CUDA_TRY(cudaEventRecord(e1, st));
    CUDA_TRY(cudaMemcpyAsync(sa_out, d_sorted, (size_t)m * 4, cudaMemcpyDeviceToHost, st));
    CUDA_TRY(cudaMemcpyAsync(lcp_out, d_lcp, (size_t)m * 4, cudaMemcpyDeviceToHost, st));
    CUDA_TRY(cudaStreamSynchronize(st));
    if (device_ms_out) CUDA_TRY(cudaEventElapsedTime(device_ms_out, e0, e1));
done:
    cudaFree(d_corpus);
    cudaFree(d_sa0);
    cudaFree(d_sa1);
    cudaFree(d_lcp);
    if (e0) cudaEventDestroy(e0);
    if (e1) cudaEventDestroy(e1);
    if (st) cudaStreamDestroy(st);
    return rc;
}

extern "C" int agpt_b200_trie_build_gpu(const int32_t *corpus, int64_t n, int max_depth, int subtree_level, int prune_min_mass,
                                        int prune_min_depth, int device, agpt_trie **out) {
    if (!corpus || !out || max_depth < 1) return agpt_set_error(AGPT_E_ARG, "trie_build_gpu: bad argument");
    if (n < (int64_t)max_depth + 2) return agpt_set_error(AGPT_E_ARG, "trie_build_gpu: corpus shorter than max_depth + 2 tokens");
    std::vector<int32_t> sa((size_t)(n - 1)), lcp((size_t)(n - 1));
    int rc = agpt_b200_suffix_order_gpu(corpus, n, max_depth + 1, device, sa.data(), lcp.data(), nullptr);
    if (rc) return rc;
    return agpt_b200_trie_from_suffix_order(corpus, n, max_depth, subtree_level, prune_min_mass, prune_min_depth, sa.data(), lcp.data(), out);
}
