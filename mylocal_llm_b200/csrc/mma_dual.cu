// Instantiations of the tensor-core GEMV for two weight streams of the same format
// (fused gate/up SwiGLU, plain and grouped). Mixed-format pairs use the FP32-lane kernel.
#include "mma_gemv.cuh"

namespace b200q {

using MmaKernelFn = void (*)(const MmaArgs);

template <int MODE, int NT>
static MmaKernelFn pick(int fmt) {
    switch (fmt) {
        case B200Q_Q8_0: return mma_gemv_kernel<B200Q_Q8_0, B200Q_Q8_0, MODE, NT>;
        case B200Q_Q4_K: return mma_gemv_kernel<B200Q_Q4_K, B200Q_Q4_K, MODE, NT>;
        case B200Q_Q5_K: return mma_gemv_kernel<B200Q_Q5_K, B200Q_Q5_K, MODE, NT>;
        case B200Q_Q6_K: return mma_gemv_kernel<B200Q_Q6_K, B200Q_Q6_K, MODE, NT>;
    }
    return nullptr;
}

MmaKernelFn mma_pick_dual(int mode, int fmt, int nterms) {
    if (mode == 1) return nterms == 2 ? pick<1, 2>(fmt) : pick<1, 1>(fmt);
    return nterms == 2 ? pick<2, 2>(fmt) : pick<2, 1>(fmt);
}

}  // namespace b200q
