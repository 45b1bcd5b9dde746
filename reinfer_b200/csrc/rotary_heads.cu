// What stands between a mixer's input projection and its attention, for mixers that rotate NEIGHBOURING dimensions
// (2i, 2i + 1) by position * freq[i] (the interleaved pairing; elementwise.cu holds the half-split one) - all of it
// 32-bit arithmetic on the projection's 32-bit or bfloat16 rows, rounded once on the way out:
//
//  * rb_rotary_heads_append   x [T, q | k | v | ...]: + bias, rotation of the first `rot` dimensions of every q and k
//                             head with a factor on cosine and sine, values optionally mixed with the values that an
//                             earlier layer left for the same tokens (v <- (1 - lambda) v + lambda v_first), q ->
//                             [T, QH, dk], k and v into the token's cache slot (value heads of their own size)
//  * rb_latent_prep           x [T, a | c | r]: RMS norm (plain weight) of a -> [T, |a|]; RMS norm of c and the rotation of
//                             r -> the token's cache slot [c | r] of a one-head cache that holds keys only
//  * rb_rotate_pairs          a strided block of heads: rotation of the first `rot` of `width` dimensions, the rest copied
//  * rb_heads_linear          y[t, h, :] = W[h] x[t, h, :] for every head, W [H, out, in]: the plain form (one warp per
//                             output, ascending sums: a token's result does not depend on the batch); optionally
//                             times the sigmoid of a gate row
//
// Angles are float(position) * freq[i] in 32-bit, cosine and sine by sincosf (no fast-math).
#include "common.cuh"

#define RH_WARPS 4

__device__ __forceinline__ void rh_rotate(float& u, float& v, int pos, float freq, float mag) {
    float sn, cs;
    sincosf((float)pos * freq, &sn, &cs);
    cs *= mag; sn *= mag;
    const float a = u * cs - v * sn, b = v * cs + u * sn;
    u = a; v = b;
}

// One warp per (token, head slot); slots: QH query heads, KH key heads, KH value heads.
template <typename TX, typename TO>
__global__ void __launch_bounds__(RH_WARPS * 32)
rotary_heads_append_kernel(const TX* __restrict__ x, long long x_stride, const float* __restrict__ bias,
                           const int* __restrict__ positions, const float* __restrict__ freq, int rot, float mag,
                           const int* __restrict__ kv_slot, TO* __restrict__ q_out, TO* __restrict__ cache,
                           int QH, int KH, int dk, int dv, int page_size, int vmix, const float* __restrict__ lambda,
                           float* __restrict__ v_first, int layout) {
    pdl_trigger();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x;
    const int slot = blockIdx.y * RH_WARPS + warp;
    if (slot >= QH + 2 * KH) return;
    const int pos = positions[t];
    pdl_wait();
    const TX* row = x + (size_t)t * x_stride;
    if (slot < QH + KH) {                                     // a query or key head: bias, rotation
        const int col0 = slot * dk;                           // q heads, then k heads, side by side
        TO* dst;
        if (slot < QH) {
            dst = q_out + ((size_t)t * QH + slot) * dk;
        } else {
            const int s = kv_slot ? kv_slot[t] : -1;
            if (s < 0) return;                                // an inert row stores nothing
            const int kh = slot - QH;
            const size_t page_stride = (size_t)KH * page_size * (dk + dv);
            dst = cache + (size_t)(s / page_size) * page_stride + (size_t)kh * page_size * dk + (size_t)(s % page_size) * dk;
        }
        if (layout == 1) {                                    // half-split pairing: dimension i turns with i + rot / 2
            const int half = rot / 2;
            for (int i = lane; i < dk; i += 32) {
                if (i < half) {
                    float u = to_f32(row[col0 + i]) + (bias ? bias[col0 + i] : 0.0f);
                    float v = to_f32(row[col0 + i + half]) + (bias ? bias[col0 + i + half] : 0.0f);
                    rh_rotate(u, v, pos, freq[i], mag);
                    dst[i] = from_f32<TO>(u);
                    dst[i + half] = from_f32<TO>(v);
                } else if (i >= rot) {
                    dst[i] = from_f32<TO>(to_f32(row[col0 + i]) + (bias ? bias[col0 + i] : 0.0f));
                }
            }
            return;
        }
        for (int p = lane; 2 * p < dk; p += 32) {
            const int i = 2 * p;
            float u = to_f32(row[col0 + i]) + (bias ? bias[col0 + i] : 0.0f);
            if (i + 1 < dk) {
                float v = to_f32(row[col0 + i + 1]) + (bias ? bias[col0 + i + 1] : 0.0f);
                if (i + 1 < rot) rh_rotate(u, v, pos, freq[p], mag);
                dst[i + 1] = from_f32<TO>(v);
            }
            dst[i] = from_f32<TO>(u);
        }
        return;
    }
    // a value head: bias, the mix with the first layer's values, store
    const int kh = slot - QH - KH;
    const int col0 = (QH + KH) * dk + kh * dv;
    const int s = kv_slot ? kv_slot[t] : -1;
    const size_t page_stride = (size_t)KH * page_size * (dk + dv);
    TO* dst = s < 0 ? nullptr : cache + (size_t)(s / page_size) * page_stride + (size_t)KH * page_size * dk +
                                    (size_t)kh * page_size * dv + (size_t)(s % page_size) * dv;
    float* vf = v_first ? v_first + ((size_t)t * KH + kh) * dv : nullptr;
    const float lam = (vmix == 2) ? lambda[0] : 0.0f;
    for (int i = lane; i < dv; i += 32) {
        float v = to_f32(row[col0 + i]) + (bias ? bias[col0 + i] : 0.0f);
        if (vmix == 1) vf[i] = v;                             // this layer's values are the ones later layers mix in
        else if (vmix == 2) v = (1.0f - lam) * v + lam * vf[i];
        if (dst) dst[i] = from_f32<TO>(v);
    }
}

// layout: 0 neighbouring pairs (2i, 2i + 1); 1 half-split pairs (i, i + rot / 2), both over the first `rot` dimensions.
// vmix: 0 none; 1 this layer leaves its values (with bias, before rounding) in v_first [T, KH * dv] float; 2 it mixes
// them in with the weight lambda[0] (a float on the device).
extern "C" int rb_rotary_heads_append(const void* x, long long x_stride, int x_dtype, const float* bias, const int* positions,
                                      const float* freq, int rot, float mag, const int* kv_slot, void* q_out, void* cache,
                                      int out_dtype, int T, int QH, int KH, int dk, int dv, int page_size, int vmix,
                                      const float* lambda, float* v_first, int layout, void* stream) {
    if (T <= 0) return 0;
    if (layout != 0 && layout != 1) RB_REFUSE("rotary_heads_append: pairing %d", layout);
    if (QH <= 0 || KH <= 0 || dk <= 0 || dv <= 0 || page_size <= 0) RB_REFUSE("rotary_heads_append: sizes %d %d %d %d %d", QH, KH, dk, dv, page_size);
    if (rot < 0 || rot % 2 || rot > dk) RB_REFUSE("rotary_heads_append: %d rotated dimensions of %d", rot, dk);
    if (rot > 0 && (!freq || !positions)) RB_REFUSE("rotary_heads_append: a rotation needs frequencies and positions");
    if (vmix < 0 || vmix > 2 || (vmix && !v_first) || (vmix == 2 && !lambda)) RB_REFUSE("rotary_heads_append: value mixing %d without its tensors", vmix);
    if (!positions) RB_REFUSE("rotary_heads_append: positions");
    cudaStream_t s = (cudaStream_t)stream;
    dim3 grid(T, rb_ceil_div(QH + 2 * KH, RH_WARPS));
#define RH_GO(TX, TO) return rb_launch(rotary_heads_append_kernel<TX, TO>, grid, dim3(RH_WARPS * 32), 0, s, (const TX*)x, x_stride, bias, \
        positions, freq, rot, mag, kv_slot, (TO*)q_out, (TO*)cache, QH, KH, dk, dv, page_size, vmix, lambda, v_first, layout)
    if (x_dtype == RB_F32 && out_dtype == RB_F32) RH_GO(float, float);
    if (x_dtype == RB_F32 && out_dtype == RB_BF16) RH_GO(float, bf16);
    if (x_dtype == RB_BF16 && out_dtype == RB_BF16) RH_GO(bf16, bf16);
#undef RH_GO
    RB_REFUSE("rotary_heads_append: dtypes %d -> %d", x_dtype, out_dtype);
}

// One CTA per token.  x row = [a: na | c: nc | r: nr].  The row comes into shared memory as floats in one pass (every
// load in flight at once: with a handful of tokens the kernel is one memory latency, not one per pass); the sums of
// squares and the outputs read it there.
#define LP_THREADS 256
template <typename TX, typename TO>
__global__ void __launch_bounds__(LP_THREADS)
latent_prep_kernel(const TX* __restrict__ x, long long x_stride, int na, int nc, int nr, const float* __restrict__ wa,
                   const float* __restrict__ wc, float eps, const int* __restrict__ positions, const float* __restrict__ freq,
                   int rot, float mag, const int* __restrict__ kv_slot, TO* __restrict__ a_out, TO* __restrict__ cache, int page_size) {
    extern __shared__ float lp_row[];
    __shared__ float red[32];
    pdl_trigger();
    const int t = blockIdx.x;
    const int pos = positions[t];
    const int s = kv_slot ? kv_slot[t] : -1;
    pdl_wait();
    const TX* row = x + (size_t)t * x_stride;
    const int n = na + nc + nr;
#pragma unroll 8
    for (int i = threadIdx.x; i < n; i += LP_THREADS) lp_row[i] = to_f32(row[i]);
    __syncthreads();
    float sa = 0.0f, sc = 0.0f;
    for (int i = threadIdx.x; i < na; i += LP_THREADS) { const float v = lp_row[i]; sa = fmaf(v, v, sa); }
    for (int i = threadIdx.x; i < nc; i += LP_THREADS) { const float v = lp_row[na + i]; sc = fmaf(v, v, sc); }
    sa = block_sum(sa, red);
    sc = block_sum(sc, red);
    const float ia = 1.0f / sqrtf(sa / (float)na + eps), ic = 1.0f / sqrtf(sc / (float)nc + eps);
    TO* ao = a_out + (size_t)t * na;
#pragma unroll 4
    for (int i = threadIdx.x; i < na; i += LP_THREADS) ao[i] = from_f32<TO>(lp_row[i] * ia * wa[i]);
    if (s < 0) return;                                        // an inert row stores nothing
    const int d = nc + nr;
    TO* dst = cache + (size_t)(s / page_size) * page_size * d + (size_t)(s % page_size) * d;
    for (int i = threadIdx.x; i < nc; i += LP_THREADS) dst[i] = from_f32<TO>(lp_row[na + i] * ic * wc[i]);
    for (int p = threadIdx.x; 2 * p < nr; p += LP_THREADS) {
        const int i = 2 * p;
        float u = lp_row[na + nc + i];
        if (i + 1 < nr) {
            float v = lp_row[na + nc + i + 1];
            if (i + 1 < rot) rh_rotate(u, v, pos, freq[p], mag);
            dst[nc + i + 1] = from_f32<TO>(v);
        }
        dst[nc + i] = from_f32<TO>(u);
    }
}

template <typename TX, typename TO>
static int lp_launch(size_t smem, int T, cudaStream_t s, const TX* x, long long x_stride, int na, int nc, int nr, const float* wa,
                     const float* wc, float eps, const int* positions, const float* freq, int rot, float mag, const int* kv_slot,
                     TO* a_out, TO* cache, int page_size) {
    static size_t allowed = 48 * 1024;
    if (smem > allowed) {
        cudaError_t e = cudaFuncSetAttribute(latent_prep_kernel<TX, TO>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        allowed = smem;
    }
    return rb_launch(latent_prep_kernel<TX, TO>, dim3(T), dim3(LP_THREADS), smem, s, x, x_stride, na, nc, nr, wa, wc, eps,
                     positions, freq, rot, mag, kv_slot, a_out, cache, page_size);
}

// wa [na], wc [nc]: float norm weights (as stored, no offset).  The cache is one layer of a one-head cache whose pages
// hold keys only: [page][page_size][nc + nr].  kv_slot null: only a_out is made.
extern "C" int rb_latent_prep(const void* x, long long x_stride, int x_dtype, int na, int nc, int nr, const float* wa, const float* wc,
                              float eps, const int* positions, const float* freq, int rot, float mag, const int* kv_slot,
                              void* a_out, void* cache, int out_dtype, int T, int page_size, void* stream) {
    if (T <= 0) return 0;
    if (na <= 0 || nc <= 0 || nr < 0 || page_size <= 0) RB_REFUSE("latent_prep: sizes %d %d %d, pages of %d", na, nc, nr, page_size);
    if (rot < 0 || rot % 2 || rot > nr) RB_REFUSE("latent_prep: %d rotated dimensions of %d", rot, nr);
    if (!positions || (rot > 0 && !freq) || !wa || !wc) RB_REFUSE("latent_prep: positions, frequencies and norm weights");
    cudaStream_t s = (cudaStream_t)stream;
    const size_t smem = (size_t)(na + nc + nr) * sizeof(float);
    if (smem > 200 * 1024) RB_REFUSE("latent_prep: a row of %d numbers does not fit shared memory", na + nc + nr);
#define LP_GO(TX, TO) return lp_launch<TX, TO>(smem, T, s, (const TX*)x, x_stride, na, nc, nr, wa, wc, eps, \
        positions, freq, rot, mag, kv_slot, (TO*)a_out, (TO*)cache, page_size)
    if (x_dtype == RB_F32 && out_dtype == RB_F32) LP_GO(float, float);
    if (x_dtype == RB_F32 && out_dtype == RB_BF16) LP_GO(float, bf16);
    if (x_dtype == RB_BF16 && out_dtype == RB_BF16) LP_GO(bf16, bf16);
#undef LP_GO
    RB_REFUSE("latent_prep: dtypes %d -> %d", x_dtype, out_dtype);
}

// One warp per (token, head): dst[t][h][0..width) = src[t][h][0..width) with the first `rot` dimensions rotated.
template <typename T>
__global__ void __launch_bounds__(RH_WARPS * 32)
rotate_pairs_kernel(const T* __restrict__ src, long long src_row, long long src_head, T* __restrict__ dst, long long dst_row,
                    long long dst_head, const int* __restrict__ positions, const float* __restrict__ freq, int H, int width, int rot, float mag) {
    pdl_trigger();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x, h = blockIdx.y * RH_WARPS + warp;
    if (h >= H) return;
    const int pos = positions[t];
    pdl_wait();
    const T* s = src + (size_t)t * src_row + (size_t)h * src_head;
    T* d = dst + (size_t)t * dst_row + (size_t)h * dst_head;
    for (int p = lane; 2 * p < width; p += 32) {
        const int i = 2 * p;
        float u = to_f32(s[i]);
        if (i + 1 < width) {
            float v = to_f32(s[i + 1]);
            if (i + 1 < rot) rh_rotate(u, v, pos, freq[p], mag);
            d[i + 1] = from_f32<T>(v);
        }
        d[i] = from_f32<T>(u);
    }
}

extern "C" int rb_rotate_pairs(const void* src, long long src_row, long long src_head, void* dst, long long dst_row, long long dst_head,
                               int dtype, const int* positions, const float* freq, int T, int H, int width, int rot, float mag, void* stream) {
    if (T <= 0 || H <= 0 || width <= 0) return 0;
    if (rot < 0 || rot % 2 || rot > width || !positions || (rot > 0 && !freq)) RB_REFUSE("rotate_pairs: %d rotated dimensions of %d", rot, width);
    cudaStream_t s = (cudaStream_t)stream;
    dim3 grid(T, rb_ceil_div(H, RH_WARPS));
    if (dtype == RB_F32)
        return rb_launch(rotate_pairs_kernel<float>, grid, dim3(RH_WARPS * 32), 0, s, (const float*)src, src_row, src_head, (float*)dst,
                         dst_row, dst_head, positions, freq, H, width, rot, mag);
    if (dtype == RB_BF16)
        return rb_launch(rotate_pairs_kernel<bf16>, grid, dim3(RH_WARPS * 32), 0, s, (const bf16*)src, src_row, src_head, (bf16*)dst,
                         dst_row, dst_head, positions, freq, H, width, rot, mag);
    RB_REFUSE("rotate_pairs: dtype %d", dtype);
}

// One CTA per (token, head): the head's input in shared memory as floats, one warp per output in turn.
template <typename TA, typename TW>
__global__ void __launch_bounds__(RH_WARPS * 32)
heads_linear_kernel(const TA* __restrict__ x, long long x_row, long long x_head, const TW* __restrict__ w, TA* __restrict__ y,
                    long long y_row, long long y_head, int n_in, int n_out, const float* __restrict__ gate, long long gate_row) {
    extern __shared__ float xs[];
    pdl_trigger(); pdl_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x, h = blockIdx.y;
    const TA* xp = x + (size_t)t * x_row + (size_t)h * x_head;
    for (int i = threadIdx.x; i < n_in; i += blockDim.x) xs[i] = to_f32(xp[i]);
    __syncthreads();
    const TW* wh = w + (size_t)h * n_out * n_in;
    TA* yp = y + (size_t)t * y_row + (size_t)h * y_head;
    for (int o = warp; o < n_out; o += RH_WARPS) {
        const TW* wr = wh + (size_t)o * n_in;
        float acc = 0.0f;
        for (int i = lane; i < n_in; i += 32) acc = fmaf(xs[i], to_f32(wr[i]), acc);
        acc = warp_sum(acc);
        if (lane == 0) {
            if (gate) acc *= 1.0f / (1.0f + expf(-gate[(size_t)t * gate_row + (size_t)h * n_out + o]));
            yp[o] = from_f32<TA>(acc);
        }
    }
}

// x [T, H, n_in] and y [T, H, n_out] with row and head strides of their own (in elements); w [H, n_out, n_in] contiguous.
// gate (null: none): float rows [T, >= H * n_out] with stride gate_row; y is multiplied by sigmoid(gate[t, h * n_out + o]).
extern "C" int rb_heads_linear(const void* x, long long x_row, long long x_head, int a_dtype, const void* w, int w_dtype, void* y,
                               long long y_row, long long y_head, int T, int H, int n_in, int n_out, const float* gate,
                               long long gate_row, void* stream) {
    if (T <= 0 || H <= 0 || n_out <= 0) return 0;
    if (n_in <= 0 || n_in > 12288) RB_REFUSE("heads_linear: %d inputs a head (supported: 1..12288)", n_in);
    cudaStream_t s = (cudaStream_t)stream;
    const size_t smem = (size_t)n_in * sizeof(float);
    dim3 grid(T, H);
#define HL_GO(TA, TW) return rb_launch(heads_linear_kernel<TA, TW>, grid, dim3(RH_WARPS * 32), smem, s, (const TA*)x, x_row, x_head, (const TW*)w, \
        (TA*)y, y_row, y_head, n_in, n_out, gate, gate_row)
    if (a_dtype == RB_F32 && w_dtype == RB_F32) HL_GO(float, float);
    if (a_dtype == RB_BF16 && w_dtype == RB_BF16) HL_GO(bf16, bf16);
    if (a_dtype == RB_BF16 && w_dtype == RB_F32) HL_GO(bf16, float);
#undef HL_GO
    RB_REFUSE("heads_linear: dtypes %d, %d", a_dtype, w_dtype);
}
