// Host-side plumbing shared by all entry points: error text, device status word, SM count.
#include <cstdarg>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <mutex>

#include "common.cuh"

namespace b200q {

static thread_local char g_error[512] = "";

void set_error(const char *fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, ap);
    va_end(ap);
}

int fail(int rc, const char *fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, ap);
    va_end(ap);
    return rc;
}

int check_launch(const char *what) {
    cudaError_t err = cudaPeekAtLastError();
    if (err != cudaSuccess) {
        cudaGetLastError();
        return fail(B200Q_ECUDA, "%s: %s", what, cudaGetErrorString(err));
    }
    return B200Q_OK;
}

// Environment switch of the programmatic dependent launches (read at every launch so a test can
// flip it): B200Q_CHAIN=0 launches every kernel with the usual full stream serialisation.
bool chain_enabled() {
    const char *v = std::getenv("B200Q_CHAIN");
    return !(v && std::strcmp(v, "0") == 0);
}

// One status word per device, living in a __device__ variable so no allocation is needed.
__device__ int g_status_word;

int *device_status_word() {
    static std::mutex mu;
    static int *ptrs[64] = {nullptr};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return nullptr;
    std::lock_guard<std::mutex> lock(mu);
    if (!ptrs[dev]) {
        void *p = nullptr;
        if (cudaGetSymbolAddress(&p, g_status_word) != cudaSuccess) {
            cudaGetLastError();
            return nullptr;
        }
        ptrs[dev] = static_cast<int *>(p);
    }
    return ptrs[dev];
}

int sm_count() {
    static int counts[64] = {0};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return NUM_SMS_FALLBACK;
    if (!counts[dev]) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) {
            cudaGetLastError();
            n = NUM_SMS_FALLBACK;
        }
        counts[dev] = n;
    }
    return counts[dev];
}

}  // namespace b200q

extern "C" {

int b200q_abi_version(void) { return 1; }

const char *b200q_last_error(void) { return b200q::g_error; }

int b200q_device_status(int *status_out) {
    if (!status_out) return b200q::fail(B200Q_EINVAL, "status_out is NULL");
    int *word = b200q::device_status_word();
    if (!word) return b200q::fail(B200Q_ECUDA, "no CUDA device / status word");
    cudaError_t err = cudaMemcpy(status_out, word, sizeof(int), cudaMemcpyDeviceToHost);
    if (err != cudaSuccess) return b200q::fail(B200Q_ECUDA, "status read: %s", cudaGetErrorString(err));
    return B200Q_OK;
}

int b200q_device_status_clear(void) {
    int *word = b200q::device_status_word();
    if (!word) return b200q::fail(B200Q_ECUDA, "no CUDA device / status word");
    cudaError_t err = cudaMemset(word, 0, sizeof(int));
    if (err != cudaSuccess) return b200q::fail(B200Q_ECUDA, "status clear: %s", cudaGetErrorString(err));
    return B200Q_OK;
}

}  // extern "C"
