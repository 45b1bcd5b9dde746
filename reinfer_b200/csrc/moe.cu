// A mixture of small feed-forward experts, the parts that are not matrix products:
//   * the router's choice: softmax over the router's outputs, the `top` largest of (score + correction) are
//     chosen, their weights are the scores themselves (not renormalised).  The last outputs may stand for
//     experts that are the identity.  The result is dense: gates [T, experts] (zero where an expert was not
//     chosen) and, per token, the sum of the chosen identity experts' scores.
//     mode 1: the vector added to the router's outputs is a bias of the logits; the `top` largest logits are chosen and
//     their weights are the softmax over the chosen logits alone.
//   * the experts' activation with the gate folded in: act[t, e*ff + c] = act(u[t, e*ff + c]) * gates[t, e]
//     (squared relu), so that ONE product with the experts' down matrices side by side gives the weighted sum of
//     the chosen experts - an expert that was not chosen contributes exact zeros.
//   * dst[t,:] (+)= a[t] * src[t,:], the identity experts' share.
// All arithmetic is 32-bit.  A token's result depends on its own row only.
#include "common.cuh"

#define ROUTE_WARPS 4

// One warp's choice for its token: score [n] holds the router's outputs and becomes the softmax over them; choice [n]
// is scratch.  Writes the token's row of gates and its identity weight.
__device__ __forceinline__ void moe_choose(float* score, float* choice, const float* __restrict__ corr, float* __restrict__ gates,
                                           float* __restrict__ ident, int t, int n, int E, int top, int lane, int mode) {
    if (mode == 1) {
        // logits with their bias; the largest are chosen one by one (the first of equal values), then softmaxed alone
        for (int i = lane; i < n; i += 32) { const float z = score[i] + (corr ? corr[i] : 0.0f); score[i] = z; choice[i] = z; }
        for (int i = lane; i < E; i += 32) gates[(size_t)t * E + i] = 0.0f;
        __syncwarp();
        float zmax = 0.0f, sum = 0.0f;
        for (int k = 0; k < top; ++k) {
            float best = -INFINITY;
            int at = 0x7fffffff;
            for (int i = lane; i < n; i += 32) {
                const float c = choice[i];
                if (c > best) { best = c; at = i; }
            }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                const float ob = __shfl_xor_sync(0xffffffffu, best, o);
                const int oa = __shfl_xor_sync(0xffffffffu, at, o);
                if (ob > best || (ob == best && oa < at)) { best = ob; at = oa; }
            }
            if (at >= n) break;
            if (k == 0) zmax = best;
            const float e = expf(best - zmax);
            sum += e;                                            // every lane holds the same values: one order for all
            if (lane == 0) {
                choice[at] = -INFINITY;
                if (at < E) gates[(size_t)t * E + at] = e;
            }
            __syncwarp();
        }
        const float inv = 1.0f / sum;
        for (int i = lane; i < E; i += 32) gates[(size_t)t * E + i] *= inv;
        if (ident && lane == 0) ident[t] = 0.0f;
        return;
    }
    float m = -INFINITY;
    for (int i = lane; i < n; i += 32) m = fmaxf(m, score[i]);
    m = warp_max(m);
    float sum = 0.0f;
    for (int i = lane; i < n; i += 32) { const float e = expf(score[i] - m); score[i] = e; sum += e; }
    sum = warp_sum(sum);
    const float inv = 1.0f / sum;
    for (int i = lane; i < n; i += 32) {
        const float s = score[i] * inv;
        score[i] = s;
        choice[i] = s + (corr ? corr[i] : 0.0f);
    }
    for (int i = lane; i < E; i += 32) gates[(size_t)t * E + i] = 0.0f;
    __syncwarp();
    float idw = 0.0f;
    for (int k = 0; k < top; ++k) {
        float best = -INFINITY;
        int at = 0x7fffffff;
        for (int i = lane; i < n; i += 32) {
            const float c = choice[i];
            if (c > best) { best = c; at = i; }                // ascending i: the first of equal values
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oa = __shfl_xor_sync(0xffffffffu, at, o);
            if (ob > best || (ob == best && oa < at)) { best = ob; at = oa; }
        }
        if (at >= n) break;                                    // nothing comparable is left
        if (lane == 0) {
            choice[at] = -INFINITY;
            if (at < E) gates[(size_t)t * E + at] = score[at];
        }
        if (at >= E) idw += score[at];
        __syncwarp();
    }
    if (ident && lane == 0) ident[t] = idw;
}

// z [T, n] float router outputs; corr [n] float (null: none); gates [T, E] float; ident [T] float (null if n == E)
__global__ void __launch_bounds__(ROUTE_WARPS * 32)
moe_route_kernel(const float* __restrict__ z, const float* __restrict__ corr, float* __restrict__ gates,
                 float* __restrict__ ident, int T, int n, int E, int top, int mode) {
    extern __shared__ float sm[];                              // per warp: scores [n], choice [n]
    pdl_trigger(); pdl_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x * ROUTE_WARPS + warp;
    if (t >= T) return;                                        // no block-wide barrier below
    float* score = sm + (size_t)warp * 2 * n;
    const float* zr = z + (size_t)t * n;
    for (int i = lane; i < n; i += 32) score[i] = zr[i];
    __syncwarp();
    moe_choose(score, score + n, corr, gates, ident, t, n, E, top, lane, mode);
}

extern "C" int rb_moe_route(const float* z, const float* corr, float* gates, float* ident, int T, int n, int E, int top,
                            int mode, void* stream) {
    if (T <= 0) return 0;
    if (n <= 0 || E < 0 || E > n || top <= 0 || top > n) RB_REFUSE("moe_route: %d outputs, %d experts, top %d", n, E, top);
    if (n > E && !ident) RB_REFUSE("moe_route: identity experts need a place for their weights");
    const size_t smem = (size_t)ROUTE_WARPS * 2 * n * sizeof(float);
    if (smem > 48 * 1024) RB_REFUSE("moe_route: %d router outputs", n);
    return rb_launch(moe_route_kernel, dim3(rb_ceil_div(T, ROUTE_WARPS)), dim3(ROUTE_WARPS * 32), smem, (cudaStream_t)stream,
                     z, corr, gates, ident, T, n, E, top, mode);
}

// The router's product and its choice in one kernel: z = x W^T in 32-bit, then the same choice.  A CTA takes
// ROUTER_TOKENS tokens (a weight vector fetched once serves them all) and eight outputs at a time; its threads share
// the row's columns in 16-byte pieces with every load of a pass in flight at once; the threads' sums meet in a warp
// butterfly and then in warp order.  A token's outputs depend on the width alone, never on the batch.
// x [T, h], W [n, h]: bfloat16 or float.
#define ROUTER_TOKENS 4
#define ROUTER_THREADS 128

__device__ __forceinline__ void moe_load8(const bf16* p, float (&v)[8]) {
    const uint4 raw = *reinterpret_cast<const uint4*>(p);
    const __nv_bfloat162* h2 = reinterpret_cast<const __nv_bfloat162*>(&raw);
#pragma unroll
    for (int i = 0; i < 4; ++i) { const float2 f = __bfloat1622float2(h2[i]); v[2 * i] = f.x; v[2 * i + 1] = f.y; }
}
__device__ __forceinline__ void moe_load8(const float* p, float (&v)[8]) {
    const float4 a = *reinterpret_cast<const float4*>(p), b = *reinterpret_cast<const float4*>(p + 4);
    v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w; v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
}

template <typename TX, typename TW>
__global__ void __launch_bounds__(ROUTER_THREADS)
moe_router_kernel(const TX* __restrict__ x, const TW* __restrict__ w, const float* __restrict__ corr, float* __restrict__ gates,
                  float* __restrict__ ident, int T, int h, int n, int E, int top, int vec, int mode) {
    extern __shared__ float sm[];                              // per token: scores [n], choice [n]
    __shared__ float part[ROUTER_THREADS / 32][ROUTER_TOKENS][8];
    pdl_trigger(); pdl_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t0 = blockIdx.x * ROUTER_TOKENS;
    const int nt = min(ROUTER_TOKENS, T - t0);
    for (int o0 = 0; o0 < n; o0 += 8) {
        const int live = min(8, n - o0);
        float acc[ROUTER_TOKENS][8];
#pragma unroll
        for (int a = 0; a < ROUTER_TOKENS; ++a)
#pragma unroll
            for (int j = 0; j < 8; ++j) acc[a][j] = 0.0f;
        if (vec) {
            for (int k = threadIdx.x * 8; k < h; k += ROUTER_THREADS * 8) {
                float xv[ROUTER_TOKENS][8];
#pragma unroll
                for (int a = 0; a < ROUTER_TOKENS; ++a) moe_load8(x + (size_t)(t0 + (a < nt ? a : 0)) * h + k, xv[a]);
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    if (j < live) {
                        float wv[8];
                        moe_load8(w + (size_t)(o0 + j) * h + k, wv);
#pragma unroll
                        for (int a = 0; a < ROUTER_TOKENS; ++a)
#pragma unroll
                            for (int i = 0; i < 8; ++i) acc[a][j] = fmaf(xv[a][i], wv[i], acc[a][j]);
                    }
                }
            }
        } else {
            for (int k = threadIdx.x; k < h; k += ROUTER_THREADS) {
#pragma unroll
                for (int j = 0; j < 8; ++j) {
                    if (j < live) {
                        const float wv = to_f32(w[(size_t)(o0 + j) * h + k]);
#pragma unroll
                        for (int a = 0; a < ROUTER_TOKENS; ++a)
                            acc[a][j] = fmaf(to_f32(x[(size_t)(t0 + (a < nt ? a : 0)) * h + k]), wv, acc[a][j]);
                    }
                }
            }
        }
#pragma unroll
        for (int a = 0; a < ROUTER_TOKENS; ++a)
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                const float v = warp_sum(acc[a][j]);
                if (lane == 0) part[warp][a][j] = v;
            }
        __syncthreads();
        if (threadIdx.x < ROUTER_TOKENS * 8) {
            const int a = threadIdx.x / 8, j = threadIdx.x % 8;
            if (j < live) {
                float v = part[0][a][j];
#pragma unroll
                for (int q = 1; q < ROUTER_THREADS / 32; ++q) v += part[q][a][j];
                sm[(size_t)a * 2 * n + o0 + j] = v;
            }
        }
        __syncthreads();
    }
    if (warp < nt) {
        float* score = sm + (size_t)warp * 2 * n;
        moe_choose(score, score + n, corr, gates, ident, t0 + warp, n, E, top, lane, mode);
    }
}

extern "C" int rb_moe_router(const void* x, int x_dtype, const void* w, int w_dtype, const float* corr, float* gates, float* ident,
                             int T, int h, int n, int E, int top, int mode, void* stream) {
    if (T <= 0) return 0;
    if (h <= 0 || n <= 0 || E < 0 || E > n || top <= 0 || top > n) RB_REFUSE("moe_router: width %d, %d outputs, %d experts, top %d", h, n, E, top);
    if (n > E && !ident) RB_REFUSE("moe_router: identity experts need a place for their weights");
    static_assert(ROUTER_TOKENS <= ROUTER_THREADS / 32, "a warp per token makes the choice");
    const size_t smem = (size_t)ROUTER_TOKENS * 2 * n * sizeof(float);
    if (smem > 40 * 1024) RB_REFUSE("moe_router: %d router outputs", n);
    cudaStream_t s = (cudaStream_t)stream;
    const int vec = h % 8 == 0 && (((uintptr_t)x | (uintptr_t)w) & 15) == 0;
    dim3 grid(rb_ceil_div(T, ROUTER_TOKENS)), block(ROUTER_THREADS);
#define RB_MR(TX, TW) return rb_launch(moe_router_kernel<TX, TW>, grid, block, smem, s, (const TX*)x, (const TW*)w, corr, gates, ident, T, h, n, E, top, vec, mode)
    if (x_dtype == RB_F32 && w_dtype == RB_F32) RB_MR(float, float);
    if (x_dtype == RB_BF16 && w_dtype == RB_BF16) RB_MR(bf16, bf16);
    if (x_dtype == RB_BF16 && w_dtype == RB_F32) RB_MR(bf16, float);
    if (x_dtype == RB_F32 && w_dtype == RB_BF16) RB_MR(float, bf16);
#undef RB_MR
    RB_REFUSE("moe_router: dtypes %d, %d", x_dtype, w_dtype);
}

// act[t, c] = relu(u[t, c])^2 * gates[t, c / ff]
template <typename TA>
__global__ void relu2_gate_kernel(const TA* __restrict__ u, const float* __restrict__ gates, TA* __restrict__ act,
                                  int T, int E, int ff) {
    pdl_trigger(); pdl_wait();
    const int width = E * ff;
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= width) return;
    for (int t = blockIdx.y; t < T; t += gridDim.y) {
        const float g = gates[(size_t)t * E + c / ff];
        float v = 0.0f;
        if (g != 0.0f) {
            const float r = fmaxf(to_f32(u[(size_t)t * width + c]), 0.0f);
            v = r * r * g;
        }
        act[(size_t)t * width + c] = from_f32<TA>(v);
    }
}

// The same over bfloat16 rows whose experts' inner width is a multiple of 8: a thread takes 16 bytes (eight columns of
// one expert) at a time, in a grid-stride loop over all tokens' columns.
__global__ void relu2_gate_vec_kernel(const bf16* __restrict__ u, const float* __restrict__ gates, bf16* __restrict__ act,
                                      long long n_vec, int E, int ff) {
    pdl_trigger(); pdl_wait();
    const int vec_per_row = E * ff / 8;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < n_vec; i += (long long)gridDim.x * blockDim.x) {
        const long long t = i / vec_per_row;
        const int c = (int)(i - t * vec_per_row) * 8;
        const float g = gates[t * E + c / ff];
        uint4 out = make_uint4(0, 0, 0, 0);
        if (g != 0.0f) {
            const uint4 in = *reinterpret_cast<const uint4*>(u + i * 8);
            const __nv_bfloat162* p = reinterpret_cast<const __nv_bfloat162*>(&in);
            __nv_bfloat162* q = reinterpret_cast<__nv_bfloat162*>(&out);
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const float2 v = __bfloat1622float2(p[j]);
                const float a0 = fmaxf(v.x, 0.0f), a1 = fmaxf(v.y, 0.0f);
                q[j] = __floats2bfloat162_rn(a0 * a0 * g, a1 * a1 * g);
            }
        }
        *reinterpret_cast<uint4*>(act + i * 8) = out;
    }
}

extern "C" int rb_relu2_gate(const void* u, const float* gates, void* act, int dtype, int T, int E, int ff, void* stream) {
    if (T <= 0 || E <= 0) return 0;
    if (ff <= 0) RB_REFUSE("relu2_gate: inner width %d", ff);
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == RB_BF16 && ff % 8 == 0 && (((uintptr_t)u | (uintptr_t)act) & 15) == 0) {
        const long long n_vec = (long long)T * E * ff / 8;
        const int blocks = (int)(n_vec / 256 + 1 < 148 * 16 ? n_vec / 256 + 1 : 148 * 16);
        return rb_launch(relu2_gate_vec_kernel, dim3(blocks), dim3(256), 0, s, (const bf16*)u, gates, (bf16*)act, n_vec, E, ff);
    }
    dim3 grid(rb_ceil_div((long long)E * ff, 256), T < 65535 ? T : 65535);
    if (dtype == RB_F32) return rb_launch(relu2_gate_kernel<float>, grid, dim3(256), 0, s, (const float*)u, gates, (float*)act, T, E, ff);
    if (dtype == RB_BF16) return rb_launch(relu2_gate_kernel<bf16>, grid, dim3(256), 0, s, (const bf16*)u, gates, (bf16*)act, T, E, ff);
    RB_REFUSE("relu2_gate: dtype %d", dtype);
}

// dst[t,:] = a[t] * src[t,:] (store) or dst[t,:] += a[t] * src[t,:]
template <typename TS>
__global__ void rows_axpy_kernel(float* __restrict__ dst, const float* __restrict__ a, const TS* __restrict__ src, int T, int h, int store) {
    pdl_trigger(); pdl_wait();
    const int c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= h) return;
    for (int t = blockIdx.y; t < T; t += gridDim.y) {
        const float v = a[t] * to_f32(src[(size_t)t * h + c]);
        float* d = dst + (size_t)t * h + c;
        *d = store ? v : *d + v;
    }
}

extern "C" int rb_rows_axpy(float* dst, const float* a, const void* src, int src_dtype, int T, int h, int store, void* stream) {
    if (T <= 0 || h <= 0) return 0;
    cudaStream_t s = (cudaStream_t)stream;
    dim3 grid(rb_ceil_div(h, 256), T < 65535 ? T : 65535);
    if (src_dtype == RB_F32) return rb_launch(rows_axpy_kernel<float>, grid, dim3(256), 0, s, dst, a, (const float*)src, T, h, store);
    if (src_dtype == RB_BF16) return rb_launch(rows_axpy_kernel<bf16>, grid, dim3(256), 0, s, dst, a, (const bf16*)src, T, h, store);
    RB_REFUSE("rows_axpy: dtype %d", src_dtype);
}
