// Entry points of the float32-accurate tensor-core GEMM for the dense projections around the trie attention
// (replaces the reference's cublasSgemm calls, src/cuda/agpt_train.cu:4675-4683, :4752, :4766-4771, :4803,
// :4840-5061), and its second implementation.  Implementation 1 (default) is the tcgen05 kernel in gemm_sm100.cu;
// implementation 0, in this file, runs on mma.sync and also serves the cases the first does not take (a general
// source matrix, the tail of a sliced reduction).  Here CUTLASS's "fast accurate" TF32 operator splits both operands into big and small TF32
// parts and issues three tensor-core MMAs per product (the same compensation the attention kernels use), so
// results agree with an IEEE float32 GEMM to about 1e-6 relative while running on mma.sync instead of the FP32
// FMA pipe.  All matrices are row-major; op(A) is A or A^T, op(B) is B or B^T:
//     out[M, N] = act(alpha * op(A)[M, K] * op(B)[K, N] + beta * C + bias row)
// The reduction over K can be cut into slices (weight gradients need that: their K is the number of trie
// positions).  Slices run as one batched GEMM into partial matrices in the workspace and a second small kernel
// adds them in slice order, so the result is repeatable bit for bit and no thread block waits on another.
#include <cuda_runtime.h>

#include <cstdlib>

#include "../../include/agpt_b200.h"
#include "internal.h"

#ifdef AGPT_NO_CUTLASS
// Built without the CUTLASS headers: the entry points exist and report that.
extern "C" int64_t agpt_b200_gemm_f32_workspace_bytes(int, int, int, int, int, int) {
    return agpt_set_error(AGPT_E_ARG, "gemm_f32: this build of the library has no CUTLASS headers");
}
extern "C" int agpt_b200_gemm_f32(int, int, int, int, int, float, const float *, int, const float *, int, float, const float *, int,
                                  const float *, int, float *, int, int, void *, int64_t, void *) {
    return agpt_set_error(AGPT_E_ARG, "gemm_f32: this build of the library has no CUTLASS headers");
}
extern "C" int agpt_b200_set_gemm_impl(int) { return agpt_set_error(AGPT_E_ARG, "gemm_f32: this build of the library has no CUTLASS headers"); }
#else

#include "cutlass/cutlass.h"
#include "cutlass/gemm/device/gemm_universal.h"

namespace {

template <typename LayoutA, typename LayoutB>
using Gemm3x = cutlass::gemm::device::GemmUniversal<
    float, LayoutA, float, LayoutB, float, cutlass::layout::RowMajor, float, cutlass::arch::OpClassTensorOp,
    cutlass::arch::Sm80, cutlass::gemm::GemmShape<128, 64, 16>, cutlass::gemm::GemmShape<64, 32, 16>,
    cutlass::gemm::GemmShape<16, 8, 8>, cutlass::epilogue::thread::LinearCombination<float, 4, float, float>,
    cutlass::gemm::threadblock::GemmIdentityThreadblockSwizzle<>, 3, 4, 4, cutlass::arch::OpMultiplyAddFastF32>;

using Row = cutlass::layout::RowMajor;
using Col = cutlass::layout::ColumnMajor;

// K rows per slice: a multiple of 4 so that every slice starts on a 16-byte boundary; the tail that the slices
// do not cover is added by one more GEMM
int slice_len(int K, int split_k) { return (K / split_k) & ~3; }

template <typename G>
int launch(const typename G::Arguments &args, cudaStream_t st) {
    G op;
    cutlass::Status s = op.can_implement(args);
    if (s != cutlass::Status::kSuccess)
        return agpt_set_error(AGPT_E_ARG, "gemm_f32: unsupported shape or alignment (%s); leading dimensions and pointers must be multiples of 4 floats",
                              cutlass::cutlassGetStatusString(s));
    if (G::get_workspace_size(args) != 0) return agpt_set_error(AGPT_E_ARG, "gemm_f32: unexpected CUTLASS workspace");
    s = op.initialize(args, nullptr, st);
    if (s != cutlass::Status::kSuccess) return agpt_set_error(AGPT_E_CUDA, "gemm_f32: initialize: %s", cutlass::cutlassGetStatusString(s));
    s = op.run(st);
    if (s != cutlass::Status::kSuccess) return agpt_set_error(AGPT_E_CUDA, "gemm_f32: run: %s", cutlass::cutlassGetStatusString(s));
    return AGPT_OK;
}

// out = sum over slices (in slice order) of part[s] + beta * C
__global__ void __launch_bounds__(256) sum_slices_kernel(const float4 *__restrict__ part, int slices, int64_t mn4, int n4, float beta,
                                                          const float *__restrict__ C, int ldc, float *__restrict__ out, int ldd) {
    int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= mn4) return;
    float4 acc = part[i];
    for (int s = 1; s < slices; s++) {
        float4 p = part[(int64_t)s * mn4 + i];
        acc.x += p.x; acc.y += p.y; acc.z += p.z; acc.w += p.w;
    }
    int64_t r = i / n4;
    int c = (int)(i - r * n4) * 4;
    if (beta != 0.f) {
        float4 cv = *reinterpret_cast<const float4 *>(C + r * ldc + c);
        acc.x += beta * cv.x; acc.y += beta * cv.y; acc.z += beta * cv.z; acc.w += beta * cv.w;
    }
    *reinterpret_cast<float4 *>(out + r * ldd + c) = acc;
}

int g_gemm_impl = -1;
int gemm_impl() {
    if (g_gemm_impl < 0) {
        const char *e = getenv("AGPT_B200_GEMM_IMPL");
        g_gemm_impl = (e && e[0] == '0') ? 0 : 1;
    }
    return g_gemm_impl;
}

// out = act(out + bias): the epilogue steps implementation 0 cannot fuse (a bias row together with a source
// matrix, or the ReLU)
__global__ void __launch_bounds__(256) post_bias_relu_kernel(float *__restrict__ out, int64_t M, int N, int ldd, const float *__restrict__ bias,
                                                              int relu) {
    const int64_t total = M * N;
    for (int64_t i = (int64_t)blockIdx.x * blockDim.x + threadIdx.x; i < total; i += (int64_t)gridDim.x * blockDim.x) {
        int64_t r = i / N;
        int c = (int)(i - r * N);
        float v = out[r * ldd + c];
        if (bias) v += __ldg(bias + c);
        if (relu) v = fmaxf(v, 0.f);
        out[r * ldd + c] = v;
    }
}

struct Extra {                       // what follows the product: out = act(alpha*AB + beta*C + bias)
    float beta;
    const float *C;
    int ldc;
    const float *bias;
    int relu;
};

template <typename G, bool TA, bool TB>
int run(int M, int N, int K, float alpha, const float *A, int lda, const float *B, int ldb, const Extra &x, float *D, int ldd,
        int split_k, void *ws, int64_t ws_bytes, cudaStream_t st) {
    using Mode = cutlass::gemm::GemmUniversalMode;
    int ks = split_k > 1 ? slice_len(K, split_k) : 0;
    const bool sm100 = gemm_impl() == 1 && N % 4 == 0 && lda % 4 == 0 && ldb % 4 == 0 && ldd % 4 == 0 && (!x.C || x.ldc % 4 == 0) &&
                       (((uintptr_t)A | (uintptr_t)B | (uintptr_t)D | (uintptr_t)x.C | (uintptr_t)x.bias) & 15) == 0;
    if (ks == 0) {
        if (sm100 && agpt_gemm_sm100_takes(TA, TB, x.relu, x.C != nullptr))
            return agpt_gemm_sm100(TA, TB, M, N, K, 1, alpha, A, lda, 0, B, ldb, 0, x.bias, x.relu, x.beta, x.C, x.ldc, D, ldd, 0, st);
        // implementation 0: the source operand is C, else the bias row broadcast (leading dimension 0); what is left
        // (bias on top of a source matrix, ReLU) runs as a second pass
        const bool bias_as_source = !x.C && x.bias;
        const float *src = x.C ? x.C : (bias_as_source ? x.bias : D);
        typename G::Arguments args(Mode::kGemm, {M, N, K}, 1, {alpha, x.C ? x.beta : (bias_as_source ? 1.f : 0.f)}, A, B, src, D, 0, 0, 0, 0,
                                   (int64_t)lda, (int64_t)ldb, (int64_t)(x.C ? x.ldc : (bias_as_source ? 0 : ldd)), (int64_t)ldd);
        int rc = launch<G>(args, st);
        if (rc) return rc;
        const float *late_bias = (x.C && x.bias) ? x.bias : nullptr;
        if (late_bias || x.relu) {
            int64_t blocks = ((int64_t)M * N + 255) / 256;
            post_bias_relu_kernel<<<(unsigned)(blocks < 148 * 16 ? blocks : 148 * 16), 256, 0, st>>>(D, M, N, ldd, late_bias, x.relu);
        }
        cudaError_t e = cudaGetLastError();
        if (e != cudaSuccess) return agpt_set_error(AGPT_E_CUDA, "gemm_f32: %s", cudaGetErrorString(e));
        return AGPT_OK;
    }
    if (x.bias || x.relu) return agpt_set_error(AGPT_E_ARG, "gemm_f32: split_k takes no bias or activation");
    if (N % 4 || ldd % 4 || ((uintptr_t)ws & 15)) return agpt_set_error(AGPT_E_ARG, "gemm_f32: split_k needs N and ldd multiples of 4");
    int64_t mn = (int64_t)M * N;
    if (ws_bytes < (int64_t)split_k * mn * 4) return agpt_set_error(AGPT_E_ARG, "gemm_f32: workspace too small");
    // a slice of K is ks columns of a row-major operand, ks rows of a transposed one
    int64_t sa = TA ? (int64_t)ks * lda : ks, sb = TB ? ks : (int64_t)ks * ldb;
    float *part = (float *)ws;
    int rc;
    if (sm100) {
        rc = agpt_gemm_sm100(TA, TB, M, N, ks, split_k, alpha, A, lda, sa, B, ldb, sb, nullptr, 0, 0.f, nullptr, 0, part, N, mn, st);
    } else {
        typename G::Arguments args(Mode::kBatched, {M, N, ks}, split_k, {alpha, 0.f}, A, B, part, part, sa, sb, mn, mn, (int64_t)lda, (int64_t)ldb, (int64_t)N, (int64_t)N);
        rc = launch<G>(args, st);
    }
    if (rc) return rc;
    int64_t mn4 = mn / 4;
    sum_slices_kernel<<<(unsigned)((mn4 + 255) / 256), 256, 0, st>>>((const float4 *)part, split_k, mn4, N / 4, x.C ? x.beta : 0.f, x.C, x.ldc, D, ldd);
    int tail = K - split_k * ks;
    if (tail > 0) {
        typename G::Arguments targs(Mode::kGemm, {M, N, tail}, 1, {alpha, 1.f}, A + split_k * sa, B + split_k * sb, D, D, 0, 0, 0, 0, (int64_t)lda,
                                    (int64_t)ldb, (int64_t)ldd, (int64_t)ldd);
        rc = launch<G>(targs, st);
        if (rc) return rc;
    }
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) return agpt_set_error(AGPT_E_CUDA, "gemm_f32: %s", cudaGetErrorString(e));
    return AGPT_OK;
}

}  // namespace

extern "C" int64_t agpt_b200_gemm_f32_workspace_bytes(int trans_a, int trans_b, int M, int N, int K, int split_k) {
    if (M <= 0 || N <= 0 || K <= 0 || split_k < 1) return agpt_set_error(AGPT_E_ARG, "gemm_f32_workspace_bytes: bad argument");
    if (trans_a && trans_b) return agpt_set_error(AGPT_E_ARG, "gemm_f32: A^T * B^T is not provided");
    return (split_k > 1 && slice_len(K, split_k) > 0) ? (int64_t)split_k * M * N * 4 : 0;
}

extern "C" int agpt_b200_set_gemm_impl(int impl) {
    if (impl != 0 && impl != 1) return agpt_set_error(AGPT_E_ARG, "set_gemm_impl: 0 (mma.sync, three TF32 products) or 1 (tcgen05, bf16 splits)");
    g_gemm_impl = impl;
    return AGPT_OK;
}

extern "C" int agpt_b200_gemm_f32(int trans_a, int trans_b, int M, int N, int K, float alpha, const float *d_a, int lda,
                                  const float *d_b, int ldb, float beta, const float *d_c, int ldc, const float *d_bias, int relu,
                                  float *d_out, int ldd, int split_k, void *d_workspace, int64_t workspace_bytes, void *stream) {
    if (M <= 0 || N <= 0 || K <= 0 || split_k < 1 || !d_a || !d_b || !d_out)
        return agpt_set_error(AGPT_E_ARG, "gemm_f32: bad argument");
    if (beta != 0.f && !d_c) return agpt_set_error(AGPT_E_ARG, "gemm_f32: beta != 0 needs a source matrix");
    if (d_c && ldc < N) return agpt_set_error(AGPT_E_ARG, "gemm_f32: ldc smaller than N");
    cudaStream_t st = (cudaStream_t)stream;
    Extra x{beta, beta != 0.f ? d_c : nullptr, ldc, d_bias, relu ? 1 : 0};
    // a transposed row-major operand is the same memory read as column-major
    if (!trans_a && !trans_b) return run<Gemm3x<Row, Row>, false, false>(M, N, K, alpha, d_a, lda, d_b, ldb, x, d_out, ldd, split_k, d_workspace, workspace_bytes, st);
    if (!trans_a && trans_b) return run<Gemm3x<Row, Col>, false, true>(M, N, K, alpha, d_a, lda, d_b, ldb, x, d_out, ldd, split_k, d_workspace, workspace_bytes, st);
    if (trans_a && !trans_b) return run<Gemm3x<Col, Row>, true, false>(M, N, K, alpha, d_a, lda, d_b, ldb, x, d_out, ldd, split_k, d_workspace, workspace_bytes, st);
    return agpt_set_error(AGPT_E_ARG, "gemm_f32: A^T * B^T is not provided");
}
#endif  // AGPT_NO_CUTLASS
