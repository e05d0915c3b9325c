// Instantiations of the tensor-core GEMV for one weight stream (linear, grouped down).
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

MmaKernelFn mma_pick_single(int mode, int fmt, int nterms) {
    if (mode == 0) return nterms == 2 ? pick<0, 2>(fmt) : pick<0, 1>(fmt);
    return nterms == 2 ? pick<3, 2>(fmt) : pick<3, 1>(fmt);
}

}  // namespace b200q
