// One SwiGLU expert FFN that needs no allocator: y = down( silu(x G^T) * (x U^T) ).
//
// The two-kernel expert (fused gate/up SwiGLU, then the down projection) needs a place for the
// hidden activations between the kernels. Normally the caller's framework allocates it. Some
// callers cannot: code running inside a CUDA stream capture or a real-time serving loop where
// cudaMalloc is forbidden or would synchronise the device, and hosts that bind this library from
// a language runtime without a device allocator of their own (a plain C, Go or Java caller that
// only owns its input and output buffers). For them the hidden activations live in a fixed array
// that is part of the library image on every GPU that loads it.
#include <mutex>

#include "common.cuh"

#define B200Q_STATIC_FFN_MAX_FLOATS (8 * 16384)   // 8 tokens x d_ff up to 16384 (512 KiB per GPU)

static __device__ __align__(256) float g_ffn_hidden[B200Q_STATIC_FFN_MAX_FLOATS];

namespace b200q {

// Device address of the array on the current device. The array's name is only a host-side handle:
// its device address is looked up once per device, with that device current.
static float *static_hidden_address() {
    static std::mutex mu;
    static float *ptrs[64] = {nullptr};
    int dev = -1;
    const cudaError_t dev_err = cudaGetDevice(&dev);
    if (dev_err != cudaSuccess || dev < 0 || dev >= 64) {
        cudaGetLastError();
        if (dev_err != cudaSuccess) set_error("expert_ffn_static: cudaGetDevice failed: %s", cudaGetErrorString(dev_err));
        else set_error("expert_ffn_static: device ordinal %d is outside the 64 devices this entry point serves", dev);
        return nullptr;
    }
    std::lock_guard<std::mutex> lock(mu);
    if (!ptrs[dev]) {
        void *p = nullptr;
        cudaError_t err = cudaGetSymbolAddress(&p, g_ffn_hidden);
        if (err != cudaSuccess) {
            cudaGetLastError();
            set_error("expert_ffn_static: cudaGetSymbolAddress failed: %s", cudaGetErrorString(err));
            return nullptr;
        }
        ptrs[dev] = static_cast<float *>(p);
    }
    return ptrs[dev];
}

}  // namespace b200q

using namespace b200q;

extern "C" int b200q_expert_ffn_static(const void *gate, int gate_fmt, const void *up, int up_fmt, const void *down,
                                       int down_fmt, int d_model, int d_ff, const void *x, int x_dtype, int m,
                                       void *y, int y_dtype, void *stream) {
    if (!gate || !up || !down || !x || !y) return fail(B200Q_EINVAL, "expert_ffn_static: NULL pointer");
    if (m < 1 || d_ff < 1 || d_model < 1) return fail(B200Q_EINVAL, "expert_ffn_static: bad shape");
    // everything the two inner calls would reject is checked here, so either both kernels launch or none
    auto base_fmt = [](int fmt, bool swiglu_side) {
        if (direct_tiled_base(fmt) >= 0) return direct_tiled_base(fmt);
        if (!swiglu_side && fmt == B200Q_Q6_K_TILED) return B200Q_Q6_K;
        if (!swiglu_side && fmt == B200Q_Q8_0_TILED) return B200Q_Q8_0;
        return fmt;
    };
    const int gf = base_fmt(gate_fmt, true), uf = base_fmt(up_fmt, true), df = base_fmt(down_fmt, false);
    if (!fmt_valid(gf) || !fmt_valid(uf) || !fmt_valid(df)) return fail(B200Q_EINVAL, "expert_ffn_static: unknown format");
    if ((direct_tiled_base(gate_fmt) >= 0) != (direct_tiled_base(up_fmt) >= 0))
        return fail(B200Q_EINVAL, "expert_ffn_static: gate and up must share the layout");
    if (!dtype_valid(x_dtype) || !dtype_valid(y_dtype)) return fail(B200Q_EINVAL, "expert_ffn_static: bad element type");
    if (d_model % fmt_elems(gf) || d_model % fmt_elems(uf) || d_ff % fmt_elems(df))
        return fail(B200Q_EINVAL, "expert_ffn_static: d_model / d_ff must be multiples of the formats' block size");
    if ((gate_fmt != gf && (d_ff % 16 || d_model % 256)) || (down_fmt != df && (d_model % 16 || d_ff % 256)))
        return fail(B200Q_EINVAL, "expert_ffn_static: a tile layout needs rows in multiples of 16 and K of 256");
    if (static_cast<long long>(m) * d_ff > B200Q_STATIC_FFN_MAX_FLOATS)
        return fail(B200Q_EUNSUPPORTED,
                    "expert_ffn_static: m*d_ff = %lld exceeds the built-in scratch of %d floats; use b200q_swiglu + "
                    "b200q_gemv with a caller-owned buffer",
                    static_cast<long long>(m) * d_ff, B200Q_STATIC_FFN_MAX_FLOATS);
    float *hidden = static_hidden_address();
    if (!hidden) return B200Q_ECUDA;
    // Both kernels overwrite every element they later read, so nothing has to be cleared.
    int rc = b200q_swiglu(gate, gate_fmt, up, up_fmt, d_ff, d_model, x, x_dtype, m, hidden, B200Q_F32, stream);
    if (rc) return rc;
    return b200q_gemv(down, down_fmt, d_model, d_ff, hidden, B200Q_F32, m, y, y_dtype, stream);
}
