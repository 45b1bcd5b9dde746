// The pointwise middle of a gated feed-forward whose two first products come side by side, gu [T, gate: F | up: F]:
//
//   act[t, c] = f(gu[t, c] + b[c]) * (gu[t, F + c] + b[F + c]) * gates[t, c / ff]
//
// f: 0 silu, z sigmoid(z); 1 the tanh form of gelu, 0.5 z (1 + tanh(sqrt(2/pi) (z + 0.044715 z^3))).  The biases (float
// [2F]) and the gates (float [T, F / ff]: one factor per token and block of `ff` columns - an expert of a mixture whose
// experts' first products were stacked; zero where the expert was not chosen, and then nothing is read) are optional.
// And the row vector that a last product's bias adds to every row of the float stream.  32-bit arithmetic, one
// rounding on the way out; a token's result depends on its own row only.
#include "common.cuh"

__device__ __forceinline__ float glu_f(float z, int kind) {
    // tanh-gelu: 0.5 (1 + tanh(u)) = 1 / (1 + exp(-2u)) with u = sqrt(2/pi) (z + 0.044715 z^3): one exponential, as silu
    return z / (1.0f + expf(kind == 1 ? -1.5957691216057308f * (z + 0.044715f * z * z * z) : -z));
}

template <typename TI, typename TO>
__global__ void glu_act_kernel(const TI* __restrict__ gu, long long ld, const float* __restrict__ bias, int kind,
                               const float* __restrict__ gates, int ff, TO* __restrict__ act, int T, int F) {
    pdl_trigger(); pdl_wait();
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= F) return;
    const float bg = bias ? bias[c] : 0.0f, bu = bias ? bias[F + c] : 0.0f;
    const int E = gates ? F / ff : 0;
    for (int t = blockIdx.y; t < T; t += gridDim.y) {
        const float w = gates ? gates[(size_t)t * E + c / ff] : 1.0f;
        float v = 0.0f;
        if (w != 0.0f) {
            const TI* row = gu + (size_t)t * ld;
            v = glu_f(to_f32(row[c]) + bg, kind) * (to_f32(row[F + c]) + bu) * w;
        }
        act[(size_t)t * F + c] = from_f32<TO>(v);
    }
}

// gu [T, 2F] rows with stride ld (float or bfloat16); act [T, F] contiguous.
extern "C" int rb_glu_act(const void* gu, long long ld, int in_dtype, const float* bias, int kind, const float* gates, int ff,
                          void* act, int out_dtype, int T, int F, void* stream) {
    if (T <= 0 || F <= 0) return 0;
    if (kind != 0 && kind != 1) RB_REFUSE("glu_act: activation %d", kind);
    if (gates && (ff <= 0 || F % ff)) RB_REFUSE("glu_act: %d columns in blocks of %d", F, ff);
    cudaStream_t s = (cudaStream_t)stream;
    dim3 grid(rb_ceil_div(F, 256), T < 65535 ? T : 65535);
#define GLU_GO(TI, TO) return rb_launch(glu_act_kernel<TI, TO>, grid, dim3(256), 0, s, (const TI*)gu, ld, bias, kind, gates, ff, (TO*)act, T, F)
    if (in_dtype == RB_F32 && out_dtype == RB_F32) GLU_GO(float, float);
    if (in_dtype == RB_F32 && out_dtype == RB_BF16) GLU_GO(float, bf16);
    if (in_dtype == RB_BF16 && out_dtype == RB_BF16) GLU_GO(bf16, bf16);
#undef GLU_GO
    RB_REFUSE("glu_act: dtypes %d -> %d", in_dtype, out_dtype);
}

// x[t, :] += b for every row of the float stream; b float or bfloat16.
template <typename TB>
__global__ void add_row_vector_kernel(float* __restrict__ x, const TB* __restrict__ b, int T, int h) {
    pdl_trigger(); pdl_wait();
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= h) return;
    const float v = to_f32(b[c]);
    for (int t = blockIdx.y; t < T; t += gridDim.y) x[(size_t)t * h + c] += v;
}

extern "C" int rb_add_row_vector(float* x, const void* b, int b_dtype, int T, int h, void* stream) {
    if (T <= 0 || h <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    dim3 grid(rb_ceil_div(h, 256), T < 65535 ? T : 65535);
    if (b_dtype == RB_F32) return rb_launch(add_row_vector_kernel<float>, grid, dim3(256), 0, s, x, (const float*)b, T, h);
    if (b_dtype == RB_BF16) return rb_launch(add_row_vector_kernel<bf16>, grid, dim3(256), 0, s, x, (const bf16*)b, T, h);
    RB_REFUSE("add_row_vector: dtype %d", b_dtype);
}
