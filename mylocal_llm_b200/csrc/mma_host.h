// Request descriptor shared by the C ABI dispatcher and the tensor-core GEMV launcher.
#pragma once
#include <cuda_runtime.h>
#include <stdint.h>

namespace b200q {

struct MmaRequest {
    int mode;  // 0 linear, 1 SwiGLU, 2 grouped gate/up, 3 grouped down
    const uint8_t *wa;
    const uint8_t *wb;
    int fmt_a, fmt_b;
    long long stride_a, stride_b;
    const unsigned long long *table_a, *table_b;   // optional per-expert pointer tables
    int tables_aligned16;                          // caller vouches: every table entry is 16-byte aligned
    int tiled;                                     // Q4_K / Q5_K weights in their tile layout (direct kernel only)
    int n, k, m;
    const void *x;
    int x_dtype;
    void *y;
    int y_dtype;
    int topk;
    const int32_t *order;
    const int32_t *seg_expert;
    const int32_t *seg_begin;
    const int32_t *seg_count;
    const int32_t *num_segments;
    int max_segments;
    const float *route;
    int flat_rows;
    const uint64_t *y_table;
    int rows_per_rank;
    int *status;
    const void *images;   // mode 2, optional: per-token activation images (direct_token_images) of the rows of x
};

// Launches the tensor-core kernel when the request fits it (alignment, K multiple of 256, shared
// memory); otherwise leaves *launched false and the caller runs the FP32-lane kernel.
int mma_try_launch(const MmaRequest &q, cudaStream_t stream, bool *launched);
// Tokens per mma_try_launch() request for this format / mode / K: 8, or 16 where the direct kernel
// is in use and serves two token tiles per pass.
int mma_tokens_per_pass(int fmt, int mode, int k, int x_dtype, bool tiled);

// Same contract for the direct-load kernel (Q4_K / Q5_K only); tried first.
int direct_try_launch(const MmaRequest &q, cudaStream_t stream, bool *launched);
// Tokens per launch the direct kernel takes for this format / mode / K (8, or 16 in the dense modes
// when two token tiles fit in shared memory).
int direct_tokens_per_pass(int fmt, int mode, int k, int x_dtype);

// Activation images for the grouped gate/up launch of the direct kernel: what that kernel would prepare for
// a token (scaled FP16 fragments, sub-block sums, the scale), written once per token so that an expert
// segment only gathers its tokens' images. Bytes per token (0 = this K / dtype has no images), and the
// launch that fills `images` [rows x bytes] from x [rows x k].
int direct_token_image_bytes(int k, int x_dtype);
int direct_token_images(const void *x, int x_dtype, int rows, int k, void *images, cudaStream_t stream);

// Weights in the Q6_K / Q8_0 tile layouts (mode 0 or 3, at most tiled_tokens_per_pass() tokens):
// there is no other kernel for these layouts, so a request that does not fit returns an error
// instead of declining.
int q6k_tiled_launch(const MmaRequest &q, cudaStream_t stream);

// The kernel arguments and dynamic shared memory the two grouped launches above would use for a request,
// without launching (the persistent one-token MoE step runs the same bodies with the same split of the work).
struct DirectArgs;
struct Q6TiledArgs;
bool direct_plan_args(const MmaRequest &q, DirectArgs *out, long long *smem_out);
int tiled_plan_args(const MmaRequest &q, Q6TiledArgs *out, long long *smem_out);
int tiled_tokens_per_pass(int mode, int k, int x_dtype);

}  // namespace b200q
