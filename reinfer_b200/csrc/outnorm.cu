// The residual sum of a layer whose norm sits on the sublayer's OUTPUT:
//     x[r,:] += mult * ( y[r,:] / sqrt(mean(y[r,:]^2) + eps) ) * w        y = sum_s parts[s][r,:]
// y comes as one float row or as a stack of partial sums that a split product left (added in ascending order);
// x is the float residual stream and is updated in place.  Optionally the new x is also written rounded to
// bfloat16: the next sublayer's products read the stream itself, not a norm of it.  One CTA per row; the row of
// y lives in shared memory between the two passes.  The order of every sum depends on the width alone.
// Also here: rounding rows of the stream to bfloat16 as a kernel of its own (the first sublayer of a step).
#include "common.cuh"

template <typename TW, int VEC>
__global__ void residual_outnorm_kernel(float* __restrict__ x, const float* __restrict__ y, int n_parts, long long part_stride,
                                        const TW* __restrict__ w, bf16* __restrict__ rounded, int h, float eps, float mult,
                                        const float* __restrict__ extra_a, const void* __restrict__ extra_src, int extra_bf16,
                                        const float* __restrict__ next_w, bf16* __restrict__ next_rows, float* __restrict__ next_sumsq,
                                        int next_parts) {
    extern __shared__ __align__(16) float row[];
    __shared__ float red[32];
    pdl_trigger(); pdl_wait();
    const int r = blockIdx.x;
    const float* yr = y + (size_t)r * h;
    // an optional multiple of another row joins y before the norm: y[r,:] += extra_a[r] * extra_src[r,:]
    const float ea = extra_a ? extra_a[r] : 0.0f;
    const float* ef = (extra_a && !extra_bf16) ? (const float*)extra_src + (size_t)r * h : nullptr;
    const bf16* eb = (extra_a && extra_bf16) ? (const bf16*)extra_src + (size_t)r * h : nullptr;
    float ss = 0.0f;
    if (VEC == 4) {
        for (int i = threadIdx.x * 4; i < h; i += blockDim.x * 4) {
            float4 v = *reinterpret_cast<const float4*>(yr + i);
            for (int s0 = 1; s0 < n_parts; s0 += 8) {          // eight partial sums in flight, added in ascending order
                float4 d[8];
#pragma unroll
                for (int p = 0; p < 8; ++p)
                    d[p] = s0 + p < n_parts ? *reinterpret_cast<const float4*>(yr + (size_t)(s0 + p) * part_stride + i)
                                            : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
                for (int p = 0; p < 8; ++p) if (s0 + p < n_parts) { v.x += d[p].x; v.y += d[p].y; v.z += d[p].z; v.w += d[p].w; }
            }
            if (ef) { v.x = fmaf(ea, ef[i], v.x); v.y = fmaf(ea, ef[i + 1], v.y); v.z = fmaf(ea, ef[i + 2], v.z); v.w = fmaf(ea, ef[i + 3], v.w); }
            if (eb) { v.x = fmaf(ea, to_f32(eb[i]), v.x); v.y = fmaf(ea, to_f32(eb[i + 1]), v.y); v.z = fmaf(ea, to_f32(eb[i + 2]), v.z); v.w = fmaf(ea, to_f32(eb[i + 3]), v.w); }
            *reinterpret_cast<float4*>(row + i) = v;
            ss += v.x * v.x + v.y * v.y + v.z * v.z + v.w * v.w;
        }
    } else {
        for (int i = threadIdx.x; i < h; i += blockDim.x) {
            float v = yr[i];
            for (int s = 1; s < n_parts; ++s) v += yr[(size_t)s * part_stride + i];
            if (ef) v = fmaf(ea, ef[i], v);
            if (eb) v = fmaf(ea, to_f32(eb[i]), v);
            row[i] = v;
            ss += v * v;
        }
    }
    const float total = block_sum(ss, red);                  // (its barriers also publish `row`)
    const float f = mult / sqrtf(total / (float)h + eps);
    float* xr = x + (size_t)r * h;
    bf16* rr = rounded ? rounded + (size_t)r * h : nullptr;
    // the norm that reads the stream next, without its division: rows of x * its weight and the row's sum of squares
    bf16* nr = next_rows ? next_rows + (size_t)r * h : nullptr;
    float ss2 = 0.0f;
    if (VEC == 4) {
        for (int i = threadIdx.x * 4; i < h; i += blockDim.x * 4) {
            const float4 v = *reinterpret_cast<const float4*>(row + i);
            float4 o = *reinterpret_cast<const float4*>(xr + i);
            o.x += v.x * f * to_f32(w[i]); o.y += v.y * f * to_f32(w[i + 1]);
            o.z += v.z * f * to_f32(w[i + 2]); o.w += v.w * f * to_f32(w[i + 3]);
            *reinterpret_cast<float4*>(xr + i) = o;
            if (rr) {
                __nv_bfloat162 lo = __floats2bfloat162_rn(o.x, o.y), hi = __floats2bfloat162_rn(o.z, o.w);
                uint2 pk;
                pk.x = *reinterpret_cast<uint32_t*>(&lo); pk.y = *reinterpret_cast<uint32_t*>(&hi);
                *reinterpret_cast<uint2*>(rr + i) = pk;
            }
            if (nr) {
                const float4 nw = *reinterpret_cast<const float4*>(next_w + i);
                __nv_bfloat162 lo = __floats2bfloat162_rn(o.x * nw.x, o.y * nw.y), hi = __floats2bfloat162_rn(o.z * nw.z, o.w * nw.w);
                uint2 pk;
                pk.x = *reinterpret_cast<uint32_t*>(&lo); pk.y = *reinterpret_cast<uint32_t*>(&hi);
                *reinterpret_cast<uint2*>(nr + i) = pk;
                ss2 += o.x * o.x + o.y * o.y + o.z * o.z + o.w * o.w;
            }
        }
    } else {
        for (int i = threadIdx.x; i < h; i += blockDim.x) {
            const float o = xr[i] + row[i] * f * to_f32(w[i]);
            xr[i] = o;
            if (rr) rr[i] = __float2bfloat16_rn(o);
            if (nr) { nr[i] = __float2bfloat16_rn(o * next_w[i]); ss2 = fmaf(o, o, ss2); }
        }
    }
    if (nr) {
        const float total2 = block_sum(ss2, red);
        // (the reader adds a row's parts: the whole sum is the first, the others are zero)
        for (int p = threadIdx.x; p < next_parts; p += blockDim.x) next_sumsq[(size_t)r * next_parts + p] = p == 0 ? total2 : 0.0f;
    }
}

// y: n_parts stacked [rows, h] float arrays, part_stride elements apart.  rounded: bfloat16 [rows, h] or null.
// extra_a [rows] float with extra_src [rows, h] (float or bfloat16), or neither.  next_w [h] float with next_rows
// [rows, h] bfloat16 and next_sumsq [rows, next_parts] float, or none of them: the rows of the norm that reads the
// stream next, as rb_residual_rowscale leaves them.
extern "C" int rb_residual_outnorm(float* x, const float* y, int n_parts, long long part_stride, const void* w, int w_dtype,
                                   void* rounded, int rows, int h, float eps, float mult, const float* extra_a,
                                   const void* extra_src, int extra_dtype, const float* next_w, void* next_rows,
                                   float* next_sumsq, int next_parts, void* stream) {
    if (rows <= 0) return 0;
    if ((next_w == nullptr) != (next_rows == nullptr) || (next_w == nullptr) != (next_sumsq == nullptr) || (next_w && next_parts < 1))
        RB_REFUSE("outnorm: the next norm's rows need its weight, the rows and the sums");
    if (next_w && (((uintptr_t)next_w & 15) || ((uintptr_t)next_rows & 7))) RB_REFUSE("outnorm: the next norm's operands must be aligned");
    if ((extra_a == nullptr) != (extra_src == nullptr)) RB_REFUSE("outnorm: half an extra term");
    if (h <= 0 || n_parts < 1) RB_REFUSE("outnorm: width %d, %d partial sums", h, n_parts);
    const size_t smem = (size_t)h * sizeof(float);
    if (smem > 200 * 1024) RB_REFUSE("outnorm: a row of %d floats does not fit shared memory", h);
    cudaStream_t s = (cudaStream_t)stream;
    const bool vec = h % 4 == 0 && part_stride % 4 == 0 && ((uintptr_t)x | (uintptr_t)y) % 16 == 0 && (!rounded || (uintptr_t)rounded % 8 == 0);
    // a stack of partial sums over few rows: a thread per 16 bytes of the row, so that all of a row's loads are in flight
    // at once (the order of the sums is then a function of the width and of whether the input is a stack - never of
    // the other rows)
    int threads = h >= 4096 ? 512 : (h >= 1024 ? 256 : 128);
    if (vec && n_parts > 1) { threads = ((h / 4 + 31) / 32) * 32; if (threads > 1024) threads = 1024; if (threads < 128) threads = 128; }
#define RB_ON(TW, V) do { \
        if (smem > 48 * 1024) { \
            cudaError_t e = cudaFuncSetAttribute(residual_outnorm_kernel<TW, V>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); \
            if (e != cudaSuccess) return (int)e; \
        } \
        return rb_launch(residual_outnorm_kernel<TW, V>, dim3(rows), dim3(threads), smem, s, x, y, n_parts, part_stride, \
                         (const TW*)w, (bf16*)rounded, h, eps, mult, extra_a, extra_src, extra_dtype == RB_BF16 ? 1 : 0, \
                         next_w, (bf16*)next_rows, next_sumsq, next_parts); } while (0)
    if (w_dtype == RB_F32) { if (vec) RB_ON(float, 4); else RB_ON(float, 1); }
    if (w_dtype == RB_BF16) { if (vec) RB_ON(bf16, 4); else RB_ON(bf16, 1); }
#undef RB_ON
    RB_REFUSE("outnorm: weight dtype %d", w_dtype);
}

// out[i] = bfloat16(x[i])
__global__ void round_rows_kernel(const float* __restrict__ x, bf16* __restrict__ out, size_t n) {
    pdl_trigger(); pdl_wait();
    const size_t i = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * 2;
    if (i + 1 < n) {
        const float2 v = *reinterpret_cast<const float2*>(x + i);
        *reinterpret_cast<__nv_bfloat162*>(out + i) = __floats2bfloat162_rn(v.x, v.y);
    } else if (i < n) {
        out[i] = __float2bfloat16_rn(x[i]);
    }
}
extern "C" int rb_round_rows(const float* x, void* out, long long n, void* stream) {
    if (n <= 0) return 0;
    if (((uintptr_t)x % 8) || ((uintptr_t)out % 4)) RB_REFUSE("round_rows: unaligned rows");
    return rb_launch(round_rows_kernel, dim3(rb_ceil_div(n, 512)), dim3(256), 0, (cudaStream_t)stream, x, (bf16*)out, (size_t)n);
}
