// Tensor-core partial decode kernels for the layouts other than the unstructured FP16 bitmap:
// unstructured INT4 / INT2, tiled FP16, 4:16 structured FP16, 1-of-4 structured INT4, compact INT4 / INT2.
// Same kernel template as the bitmap layout (decode_mma.cuh); only the field policy differs.
#include "decode_common.cuh"

namespace reskv {
namespace {
#include "decode_mma.cuh"

template <int GQA, class ML, int BETA>
int launch_beta(const DecodeParams& p, cudaStream_t stream) {
    const size_t smem = mma::smem_bytes<GQA, ML>(p.ck);
    auto kern = mma::decode_mma_kernel<GQA, ML, BETA>;
    // allowed once per kernel instance and device (bit mask over device ordinals), for the largest centroid table
    static unsigned long long done = 0;
    int dev = 0;
    if (int rc = check_cuda(cudaGetDevice(&dev), "cudaGetDevice")) return rc;
    if (dev < 0 || dev >= 64 || !(done >> dev & 1ull)) {
        if (int rc = check_cuda(cudaFuncSetAttribute(kern, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                     static_cast<int>(mma::smem_bytes<GQA, ML>(kMaxClusters))),
                                "cudaFuncSetAttribute(decode_mma packed)"))
            return rc;
        if (dev >= 0 && dev < 64) done |= 1ull << dev;
    }
    kern<<<p.grid, mma::kThreadsM, smem, stream>>>(p);
    return check_cuda(cudaGetLastError(), "decode_mma (packed layout) launch");
}

// up to 32 value centroids: the instance with two cluster-mass blocks
template <int GQA, class ML>
int launch(const DecodeParams& p, int, cudaStream_t stream) {
    return p.cv <= 32 ? launch_beta<GQA, ML, 2>(p, stream) : launch_beta<GQA, ML, 4>(p, stream);
}

template <int GQA>
int by_layout(const DecodeParams& p, int layout, int units, cudaStream_t s) {
    switch (layout) {
        case 0: return launch<GQA, mma::LayoutMmaQuant<4>>(p, units, s);
        case 1: return launch<GQA, mma::LayoutMmaQuant<2>>(p, units, s);
        case 2: return launch<GQA, mma::LayoutMmaTiled<64, false>>(p, units, s);
        case 3: return launch<GQA, mma::LayoutMmaTiled<32, true>>(p, units, s);
        case 5: return launch<GQA, mma::LayoutMmaCompact<4, 64>>(p, units, s);
        case 6: return launch<GQA, mma::LayoutMmaCompact<4, 32>>(p, units, s);
        case 7: return launch<GQA, mma::LayoutMmaCompact<2, 64>>(p, units, s);
        default: return launch<GQA, mma::LayoutMmaStructInt4>(p, units, s);
    }
}
}  // namespace

int launch_packed_mma(const DecodeParams& p, int layout, int gqa, int units, cudaStream_t stream) {
    return gqa == 1 ? by_layout<1>(p, layout, units, stream)
           : gqa == 4 ? by_layout<4>(p, layout, units, stream)
                      : by_layout<8>(p, layout, units, stream);
}
}  // namespace reskv
