// float32 GEMM on the fifth-generation tensor cores (tcgen05 MMAs with accumulators in tensor memory, operands
// brought in by TMA) for the dense projections around the trie attention.  Each float32 operand tile is split on
// chip into three bfloat16 matrices (x = b0 + b1 + b2 to 24 bits) and the product is rebuilt from the bf16 x bf16
// partial products with float32 accumulation, so results match an IEEE float32 GEMM to a few 1e-7 relative: the
// accuracy of the reference's cublasSgemm calls (src/cuda/agpt_train.cu:4675-4683, :4752, :4766-4771, :4803,
// :4840-5061) at several times their speed.  The kernel is CUTLASS's SM100 warp-specialised "fast FP32" mainloop
// (TMA load warp -> transform warps -> MMA warp -> epilogue warps), instantiated here for one CTA per tile
// (a cluster of one: every CTA loads its own operand tiles), a 128x128x32 tile, and three epilogues: bias row; bias row + ReLU (the first
// feed-forward projection); bias row + a source matrix (the residual stream added in the same pass).
// Measured on a B200, [1M, 128] x [128, 128]: the builder's defaults (k extent 16, all nine partial products, the
// accumulator read out of tensor memory after every k block of 16) 0.332 ms; six products 0.316 ms; six products,
// k extent 32 and a read-out every second k block 0.263 ms (3.9 TB/s of compulsory traffic).
#include <cuda_runtime.h>

#include "../../include/agpt_b200.h"
#include "internal.h"

#ifndef AGPT_NO_CUTLASS

#include "cute/tensor.hpp"
#include "cutlass/cutlass.h"
#include "cutlass/epilogue/collective/collective_builder.hpp"
#include "cutlass/epilogue/fusion/operations.hpp"
#include "cutlass/gemm/collective/collective_builder.hpp"
#include "cutlass/gemm/device/gemm_universal_adapter.h"
#include "cutlass/gemm/kernel/gemm_universal.hpp"

namespace {

using namespace cute;
using Row = cutlass::layout::RowMajor;
using Col = cutlass::layout::ColumnMajor;

enum { EPI_BIAS = 0, EPI_BIAS_RELU = 1, EPI_BIAS_SOURCE = 2 };

// The builder fixes the mainloop at all five significance bands of the 3 x 3 bf16 partial products (nine MMAs per
// k block).  The two lowest bands (a1 b2, a2 b1, a2 b2) are below 2^-24 of the product, the rounding of the float32
// accumulation itself, so the mainloop is re-instantiated with the same stage counts, layouts and copies,
// BANDS = 3 (six MMAs per k block) and a longer promotion interval: the accumulator warps read the whole
// 128 x 128 tile out of tensor memory and add it in registers once per interval, which bounds the loop when the
// interval is one k block.
#ifndef AGPT_GEMM_BANDS
#define AGPT_GEMM_BANDS 3      // 3, 4 or 5 bands of partial products (6, 8 or 9 MMAs per k block)
#endif
#ifndef AGPT_GEMM_TILE_K
#define AGPT_GEMM_TILE_K 32    // k extent of one pipeline stage (64 leaves fewer than two stages of shared memory)
#endif
#ifndef AGPT_GEMM_PROMOTE
#define AGPT_GEMM_PROMOTE 2    // k blocks (of 16) summed in tensor memory before the accumulator warps add them in registers
#endif

template <typename Built, int BANDS, int PROMOTE>
struct WithBands {
    using P0 = typename Built::DispatchPolicy;
    using Policy = cutlass::gemm::MainloopSm100TmaUmmaWarpSpecializedFastF32<
        P0::Load2TransformPipelineStageCount, P0::Transform2MmaPipelineStageCount, P0::Schedule::SchedulerPipelineStageCount,
        P0::Schedule::AccumulatorPipelineStageCount, BANDS, P0::ScalingFactor, PROMOTE, typename P0::ClusterShape,
        typename P0::AccumulatorCopyAtom, typename P0::ArchTag>;
    using type = cutlass::gemm::collective::CollectiveMma<
        Policy, typename Built::TileShape, float, typename Built::StrideA, float, typename Built::StrideB, typename Built::TiledMma,
        typename Built::GmemTiledCopyA, typename Built::SmemLayoutAtomsA, typename Built::CopyAtomsA, typename Built::TransformA,
        typename Built::GmemTiledCopyB, typename Built::SmemLayoutAtomsB, typename Built::CopyAtomsB, typename Built::TransformB>;
};

// One CTA per 128 x 128 tile, every CTA loading its own operand tiles.  (A CTA pair sharing a 256 x 128 tile, each
// CTA holding half of the B tile, measured 5-12 % faster on the row-streaming products and slower on the weight
// gradients; it is not used: the same library has to run unchanged in multi-GPU jobs, where cluster-wide operand
// loads are not wanted.)
template <typename LayoutA, typename LayoutB, int EPI = EPI_BIAS>
struct Sm100Gemm {
    using TileShape = Shape<_128, _128, Int<AGPT_GEMM_TILE_K>>;
    using ClusterShape = Shape<_1, _1, _1>;
    using EpilogueSchedule = cutlass::epilogue::TmaWarpSpecialized1Sm;
    using MainloopSchedule = cutlass::gemm::KernelTmaWarpSpecialized1SmFastFP32Sm100;
    // D = act(alpha * acc + beta * C + bias[column]); without a source matrix none is read (ElementC = void)
    using Fusion = cute::conditional_t<EPI == EPI_BIAS_RELU,
                                       cutlass::epilogue::fusion::LinCombPerColBiasEltAct<cutlass::epilogue::thread::ReLu, float, float, float, float, float, 4>,
                                       cutlass::epilogue::fusion::LinCombPerColBias<float, float, float, float, float, 4>>;
    using ElementC = cute::conditional_t<EPI == EPI_BIAS_SOURCE, float, void>;
    using Epilogue = typename cutlass::epilogue::collective::CollectiveBuilder<
        cutlass::arch::Sm100, cutlass::arch::OpClassTensorOp, TileShape, ClusterShape, cutlass::epilogue::collective::EpilogueTileAuto,
        float, float, ElementC, Row, 4, float, Row, 4, EpilogueSchedule, Fusion>::CollectiveOp;
    using Built = typename cutlass::gemm::collective::CollectiveBuilder<
        cutlass::arch::Sm100, cutlass::arch::OpClassTensorOp, float, LayoutA, 4, float, LayoutB, 4, float, TileShape, ClusterShape,
        cutlass::gemm::collective::StageCountAutoCarveout<static_cast<int>(sizeof(typename Epilogue::SharedStorage))>,
        MainloopSchedule>::CollectiveOp;
    using Mainloop = typename WithBands<Built, AGPT_GEMM_BANDS, AGPT_GEMM_PROMOTE>::type;
    using Kernel = cutlass::gemm::kernel::GemmUniversal<Shape<int, int, int, int>, Mainloop, Epilogue, void>;
    using Gemm = cutlass::gemm::device::GemmUniversalAdapter<Kernel>;
};

int sm_count_of(int dev) {
    static int cached[64] = {0};
    if (dev < 0 || dev >= 64) return cutlass::KernelHardwareInfo::query_device_multiprocessor_count(dev);
    if (!cached[dev]) cached[dev] = cutlass::KernelHardwareInfo::query_device_multiprocessor_count(dev);
    return cached[dev];
}

template <typename G>
int run(int M, int N, int K, int L, float alpha, const float *A, int64_t lda, int64_t batch_a, const float *B, int64_t ldb,
        int64_t batch_b, const float *bias, float beta, const float *C, int64_t ldc, float *D, int64_t ldd, int64_t batch_d,
        cudaStream_t st) {
    using Gemm = typename G::Gemm;
    typename Gemm::GemmKernel::StrideA dA;
    typename Gemm::GemmKernel::StrideB dB;
    typename Gemm::GemmKernel::StrideD dD;
    // of each (row, column) stride pair one entry is the compile-time 1, the other the leading dimension; the
    // third mode is the batch (a slice of K when the caller cuts the reduction)
    if constexpr (is_static<decltype(get<1>(dA))>::value) get<0>(dA) = lda; else get<1>(dA) = lda;
    get<2>(dA) = batch_a;
    if constexpr (is_static<decltype(get<1>(dB))>::value) get<0>(dB) = ldb; else get<1>(dB) = ldb;
    get<2>(dB) = batch_b;
    get<0>(dD) = ldd;
    get<2>(dD) = batch_d;
    typename Gemm::GemmKernel::StrideC dC = dD;
    get<0>(dC) = ldc;
    get<2>(dC) = 0;
    using PtrC = decltype(typename Gemm::Arguments{}.epilogue.ptr_C);
    typename Gemm::Arguments args{cutlass::gemm::GemmUniversalMode::kGemm, {M, N, K, L}, {A, dA, B, dB}, {{}, (PtrC)C, dC, D, dD}};
    args.epilogue.thread.alpha = alpha;
    args.epilogue.thread.beta = beta;
    args.epilogue.thread.bias_ptr = bias;
    int dev = 0;
    cudaGetDevice(&dev);
    // the tensor maps are encoded through the driver API, which needs the device's primary context current on
    // this host thread; a thread that has only queried the runtime so far (an autograd worker) has none yet
    cudaSetDevice(dev);
    args.hw_info.device_id = dev;
    args.hw_info.sm_count = sm_count_of(dev);
    Gemm op;
    cutlass::Status s = op.can_implement(args);
    if (s != cutlass::Status::kSuccess)
        return agpt_set_error(AGPT_E_ARG, "gemm_f32: unsupported shape or alignment (%s); leading dimensions and pointers must be multiples of 4 floats",
                              cutlass::cutlassGetStatusString(s));
    if (Gemm::get_workspace_size(args) != 0) return agpt_set_error(AGPT_E_ARG, "gemm_f32: unexpected CUTLASS workspace");
    s = op.initialize(args, nullptr, st);
    if (s != cutlass::Status::kSuccess) return agpt_set_error(AGPT_E_CUDA, "gemm_f32: initialize: %s", cutlass::cutlassGetStatusString(s));
    s = op.run(st);
    if (s != cutlass::Status::kSuccess) return agpt_set_error(AGPT_E_CUDA, "gemm_f32: run: %s", cutlass::cutlassGetStatusString(s));
    return AGPT_OK;
}

}  // namespace

// which (layout, epilogue) pairs are instantiated: every layout with the bias epilogue; the ReLU epilogue for the
// forward projection layout (A and B as stored); the source epilogue for that layout and for A * B^T (the input
// gradient of a projection accumulated onto the gradient of another one that read the same rows)
bool agpt_gemm_sm100_takes(int trans_a, int trans_b, int relu, int has_source) {
    if (trans_a && trans_b) return false;
    if (relu && has_source) return false;
    if (has_source) return !trans_a;
    return !relu || (!trans_a && !trans_b);
}

// D[l] = act(alpha * op(A[l]) * op(B[l]) + beta * C + bias), l < L; row-major storage, op as in agpt_b200_gemm_f32
int agpt_gemm_sm100(int trans_a, int trans_b, int M, int N, int K, int L, float alpha, const float *A, int64_t lda, int64_t batch_a,
                    const float *B, int64_t ldb, int64_t batch_b, const float *bias, int relu, float beta, const float *C, int64_t ldc,
                    float *D, int64_t ldd, int64_t batch_d, void *stream) {
    cudaStream_t st = (cudaStream_t)stream;
    if (!agpt_gemm_sm100_takes(trans_a, trans_b, relu, C != nullptr)) return agpt_set_error(AGPT_E_ARG, "gemm_f32: combination not instantiated");
    // a transposed row-major operand is the same memory read as column-major
    if (!trans_a && !trans_b) {
        if (relu) return run<Sm100Gemm<Row, Row, EPI_BIAS_RELU>>(M, N, K, L, alpha, A, lda, batch_a, B, ldb, batch_b, bias, 0.f, nullptr, ldd, D, ldd, batch_d, st);
        if (C) return run<Sm100Gemm<Row, Row, EPI_BIAS_SOURCE>>(M, N, K, L, alpha, A, lda, batch_a, B, ldb, batch_b, bias, beta, C, ldc, D, ldd, batch_d, st);
        return run<Sm100Gemm<Row, Row>>(M, N, K, L, alpha, A, lda, batch_a, B, ldb, batch_b, bias, 0.f, nullptr, ldd, D, ldd, batch_d, st);
    }
    if (!trans_a && trans_b) {
        if (C) return run<Sm100Gemm<Row, Col, EPI_BIAS_SOURCE>>(M, N, K, L, alpha, A, lda, batch_a, B, ldb, batch_b, bias, beta, C, ldc, D, ldd, batch_d, st);
        return run<Sm100Gemm<Row, Col>>(M, N, K, L, alpha, A, lda, batch_a, B, ldb, batch_b, bias, 0.f, nullptr, ldd, D, ldd, batch_d, st);
    }
    return run<Sm100Gemm<Col, Row>>(M, N, K, L, alpha, A, lda, batch_a, B, ldb, batch_b, bias, 0.f, nullptr, ldd, D, ldd, batch_d, st);
}
#endif  // AGPT_NO_CUTLASS
