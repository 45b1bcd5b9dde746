// The output stage of differential attention.  Every head ran two softmax maps over the same values; their outputs
// a1 and a2 (each [dv]) are combined and normalised per head:
//
//   o = a1 - lambda a2;   o <- o / sqrt(mean(o^2) + eps) * out_scale * sigmoid(gate[t, h])
//
// lambda is one number for the layer and out_scale a constant (both computed at load); the gate is optional, one float
// per token and head.  The maps' outputs lie in `a` [T, 2 H, dv] in the order the attention kernels' grouping wants:
// with G key heads and R = H / G, map m of head h = g R + r sits at row (2 g + m) R + r.  32-bit arithmetic, one
// warp per (token, head), sums in a fixed order.
#include "common.cuh"

template <typename TA>
__global__ void diff_heads_kernel(const TA* __restrict__ a, float lambda, float eps, float out_scale,
                                  const float* __restrict__ gate, long long gate_row, TA* __restrict__ out, int T, int H, int G, int dv) {
    pdl_trigger(); pdl_wait();
    const long long wg = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    if (wg >= (long long)T * H) return;
    const int t = (int)(wg / H), h = (int)(wg % H);
    const int R = H / G, g = h / R, r = h % R;
    const TA* a1 = a + ((size_t)t * 2 * H + (size_t)(2 * g) * R + r) * dv;
    const TA* a2 = a + ((size_t)t * 2 * H + (size_t)(2 * g + 1) * R + r) * dv;
    float ss = 0.0f;
    for (int i = lane; i < dv; i += 32) {
        const float o = to_f32(a1[i]) - lambda * to_f32(a2[i]);
        ss = fmaf(o, o, ss);
    }
    ss = warp_sum(ss);
    float f = out_scale / sqrtf(ss / (float)dv + eps);
    if (gate) f *= 1.0f / (1.0f + expf(-gate[(size_t)t * gate_row + h]));
    TA* dst = out + ((size_t)t * H + h) * dv;
    for (int i = lane; i < dv; i += 32) dst[i] = from_f32<TA>((to_f32(a1[i]) - lambda * to_f32(a2[i])) * f);
}

// a [T, 2H, dv] and out [T, H, dv] contiguous, one dtype; gate float rows [T, >= H] with stride gate_row, or null.
extern "C" int rb_diff_heads(const void* a, int dtype, float lambda, float eps, float out_scale, const float* gate,
                             long long gate_row, void* out, int T, int H, int G, int dv, void* stream) {
    if (T <= 0) return 0;
    if (H <= 0 || G <= 0 || H % G || dv <= 0) RB_REFUSE("diff_heads: %d heads over %d key heads, values of %d", H, G, dv);
    cudaStream_t s = (cudaStream_t)stream;
    const int blocks = rb_ceil_div((long long)T * H, 4);
    if (dtype == RB_F32) return rb_launch(diff_heads_kernel<float>, dim3(blocks), dim3(128), 0, s, (const float*)a, lambda, eps, out_scale, gate, gate_row, (float*)out, T, H, G, dv);
    if (dtype == RB_BF16) return rb_launch(diff_heads_kernel<bf16>, dim3(blocks), dim3(128), 0, s, (const bf16*)a, lambda, eps, out_scale, gate, gate_row, (bf16*)out, T, H, G, dv);
    RB_REFUSE("diff_heads: dtype %d", dtype);
}
