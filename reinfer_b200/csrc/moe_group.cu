// A mixture of experts over many tokens, the parts around the grouped products (gemm_tc.cu, rb_gemm_bf16_grouped): the
// tokens' rows are copied into one array sorted by expert, every expert's stretch padded to whole tiles of 128 rows, so
// that a tile of the products belongs to one expert and only the chosen (token, expert) pairs are computed.
//
//   rb_moe_group_plan     gates [T, E] float (zero where an expert was not chosen) -> for every chosen pair a row of the
//                         sorted array; per tile its expert; the number of tiles that hold rows; per token its rows
//                         (ascending by expert) and their weights; and the tokens' rows copied to their places
//   rb_moe_group_combine  dst[t, :] (+)= sum_j w[t, j] * y[row[t, j], :]   in ascending j, 32-bit
//
// Which row inside its expert's stretch a pair gets is decided by an atomic counter and may differ from run to run;
// nothing depends on it: a row's results depend on the row alone, and a token's rows are added in the order of the experts.
#include "common.cuh"

#define MG_TILE 128

__global__ void moe_group_count_kernel(const float* __restrict__ gates, int* __restrict__ count, int* __restrict__ pos, long long n, int E) {
    pdl_trigger(); pdl_wait();
    const long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (i >= n) return;
    if (gates[i] != 0.0f) pos[i] = atomicAdd(&count[i % E], 1);
}

// One CTA: the experts' stretches (each padded to whole tiles) one behind the other; tile_group for every tile that
// holds rows, the number of such tiles.
__global__ void moe_group_offsets_kernel(const int* __restrict__ count, int* __restrict__ seg_off, int* __restrict__ tile_group,
                                         int* __restrict__ live_tiles, int E, int max_tiles) {
    __shared__ int total_tiles;
    pdl_trigger(); pdl_wait();
    if (threadIdx.x == 0) {
        int at = 0;
        for (int e = 0; e < E; ++e) {
            seg_off[e] = at * MG_TILE;
            at += (count[e] + MG_TILE - 1) / MG_TILE;
        }
        total_tiles = at < max_tiles ? at : max_tiles;
        *live_tiles = total_tiles;
    }
    __syncthreads();
    for (int e = 0; e < E; ++e) {
        const int first = seg_off[e] / MG_TILE, n = (count[e] + MG_TILE - 1) / MG_TILE;
        for (int i = threadIdx.x; i < n; i += blockDim.x)
            if (first + i < max_tiles) tile_group[first + i] = e;
    }
}

// One warp per token: its chosen experts in ascending order -> rows, weights, and the token's row copied to each.
template <typename TX>
__global__ void moe_group_scatter_kernel(const TX* __restrict__ x, const float* __restrict__ gates, const int* __restrict__ pos,
                                         const int* __restrict__ seg_off, TX* __restrict__ xs, int* __restrict__ rows,
                                         float* __restrict__ w, int T, int E, int h, int top, int vec) {
    pdl_trigger(); pdl_wait();
    const int t = (blockIdx.x * blockDim.x + threadIdx.x) >> 5, lane = threadIdx.x & 31;
    if (t >= T) return;
    const TX* src = x + (size_t)t * h;
    int j = 0;
    for (int e = 0; e < E && j < top; ++e) {
        const float g = gates[(size_t)t * E + e];
        if (g == 0.0f) continue;
        const int row = seg_off[e] + pos[(size_t)t * E + e];
        if (lane == 0) { rows[(size_t)t * top + j] = row; w[(size_t)t * top + j] = g; }
        TX* dst = xs + (size_t)row * h;
        if (vec) {
            const uint4* s4 = reinterpret_cast<const uint4*>(src);
            uint4* d4 = reinterpret_cast<uint4*>(dst);
            for (int i = lane; i < h * (int)sizeof(TX) / 16; i += 32) d4[i] = s4[i];
        } else {
            for (int i = lane; i < h; i += 32) dst[i] = src[i];
        }
        ++j;
    }
    for (; j < top; ++j)
        if (lane == 0) { rows[(size_t)t * top + j] = -1; w[(size_t)t * top + j] = 0.0f; }
}

// gates [T, E] float; x [T, h] (bfloat16 or float).  Scratch: count [E] and pos [T, E] int.  Out: seg_off [E],
// tile_group [max_tiles], live_tiles [1], rows [T, top] int (-1: none), w [T, top] float, xs [max_tiles * 128, h].
extern "C" int rb_moe_group_plan(const void* x, int x_dtype, const float* gates, int* count, int* pos, int* seg_off, int* tile_group,
                                 int* live_tiles, int* rows, float* w, void* xs, int T, int E, int h, int top, int max_tiles,
                                 void* stream) {
    if (T <= 0) return 0;
    if (E <= 0 || h <= 0 || top <= 0 || top > E || max_tiles <= 0) RB_REFUSE("moe_group_plan: %d experts, width %d, top %d, %d tiles", E, h, top, max_tiles);
    if ((long long)max_tiles * MG_TILE < (long long)T * top + (long long)E * (MG_TILE - 1)) RB_REFUSE("moe_group_plan: %d tiles do not hold %d x %d rows of %d experts", max_tiles, T, top, E);
    cudaStream_t s = (cudaStream_t)stream;
    cudaError_t err = cudaMemsetAsync(count, 0, (size_t)E * sizeof(int), s);
    if (err != cudaSuccess) return (int)err;
    const long long n = (long long)T * E;
    int rc = rb_launch(moe_group_count_kernel, dim3(rb_ceil_div(n, 256)), dim3(256), 0, s, gates, count, pos, n, E);
    if (rc) return rc;
    rc = rb_launch(moe_group_offsets_kernel, dim3(1), dim3(256), 0, s, (const int*)count, seg_off, tile_group, live_tiles, E, max_tiles);
    if (rc) return rc;
    dim3 grid(rb_ceil_div((long long)T * 32, 256));
    if (x_dtype == RB_BF16) {
        const int vec = (h % 8 == 0) && ((((uintptr_t)x | (uintptr_t)xs) & 15) == 0);
        return rb_launch(moe_group_scatter_kernel<bf16>, grid, dim3(256), 0, s, (const bf16*)x, gates, (const int*)pos, (const int*)seg_off,
                         (bf16*)xs, rows, w, T, E, h, top, vec);
    }
    if (x_dtype == RB_F32) {
        const int vec = (h % 4 == 0) && ((((uintptr_t)x | (uintptr_t)xs) & 15) == 0);
        return rb_launch(moe_group_scatter_kernel<float>, grid, dim3(256), 0, s, (const float*)x, gates, (const int*)pos, (const int*)seg_off,
                         (float*)xs, rows, w, T, E, h, top, vec);
    }
    RB_REFUSE("moe_group_plan: dtype %d", x_dtype);
}

__global__ void moe_group_combine_kernel(float* __restrict__ dst, const float* __restrict__ y, const int* __restrict__ rows,
                                         const float* __restrict__ w, int T, int h, int top, int store) {
    pdl_trigger(); pdl_wait();
    const int t = blockIdx.y;
    const int c = (blockIdx.x * blockDim.x + threadIdx.x) * 4;
    if (c >= h) return;
    float4 acc = store ? make_float4(0.f, 0.f, 0.f, 0.f) : *reinterpret_cast<const float4*>(dst + (size_t)t * h + c);
    for (int j = 0; j < top; ++j) {
        const int row = rows[(size_t)t * top + j];
        if (row < 0) continue;
        const float g = w[(size_t)t * top + j];
        const float4 v = *reinterpret_cast<const float4*>(y + (size_t)row * h + c);
        acc.x = fmaf(g, v.x, acc.x); acc.y = fmaf(g, v.y, acc.y); acc.z = fmaf(g, v.z, acc.z); acc.w = fmaf(g, v.w, acc.w);
    }
    *reinterpret_cast<float4*>(dst + (size_t)t * h + c) = acc;
}

// dst [T, h] float (h a multiple of 4), y [rows, h] float.
extern "C" int rb_moe_group_combine(float* dst, const float* y, const int* rows, const float* w, int T, int h, int top, int store,
                                    void* stream) {
    if (T <= 0) return 0;
    if (h <= 0 || h % 4 || top <= 0) RB_REFUSE("moe_group_combine: width %d (a multiple of 4), top %d", h, top);
    if (T > 65535) RB_REFUSE("moe_group_combine: %d tokens exceed the grid", T);
    return rb_launch(moe_group_combine_kernel, dim3(rb_ceil_div(h / 4, 128), T), dim3(128), 0, (cudaStream_t)stream, dst, y, rows, w,
                     T, h, top, store);
}
