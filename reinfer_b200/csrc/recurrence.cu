// Linear recurrences over a matrix state per (request, head), token by token:
//
//   S [dk, dv] float, rows = key channels, one per request slot and head, carried from step to step.
//   form 0 (diagonal gate):        S <- diag(g) S + k v^T                              o = S^T q
//   form 1 (delta, old state):     S <- diag(g) S - (a*u)(u^T S_old) + k v^T           o = S^T q      u = k / |k|
//   form 2 (delta, gated state):   S <- diag(g) S;  S <- S + k (beta (v - S^T k))^T    o = S^T q
//
// A column of S (one value channel) evolves on its own, so the work is split by columns: a CTA owns
// RR_COLS columns of one (request, head), a column is shared by SPLIT adjacent lanes that hold RP rows
// each in registers, and the two dot products per token are completed by log2(SPLIT) shuffles in a fixed order.
// SPLIT is 4 where the state's traffic decides (a decode step: a warp then reads whole 32-byte pieces of a state
// row) and in 32-bit (one summation order, hence the same bits under every cut); long bfloat16 portions take 8 or 16
// lanes a column - a token's step is a chain of dependent instructions, and more warps with fewer rows each hide it.
// The CTA walks its request's tokens of this step in order; per tile of tokens all threads first prepare
// the token vectors in shared memory - the gate from its pre-activation, unit vectors, scales - in float:
// (a gate is held as g - 1 = expm1(ln g) and applied as S + (g - 1) S, so that a gate near 1 keeps its digits)
//   gate 0:  g = sigmoid(z)^(1/tau)                 = exp(-softplus(-z) / tau)
//   gate 1:  g = exp(-c * sigmoid(z))
//   gate 2:  g = exp(-exp(rate[h]) * softplus(z))
// Everything that enters the recurrence besides the projections is 32-bit; the sequence of operations for
// a token does not depend on how the request was cut into steps or on the batch.
// For portions longer than one tile the preparation runs ahead as a kernel of its own, one warp per (token, head)
// over the whole step in parallel, and leaves the vectors in a scratch buffer that the walking CTAs copy tile by
// tile: the transcendental work then stands neither in the sequential path nor is it repeated by the CTAs that
// share a head.  Both ways run the same preparation code and give the same bits.
#include "common.cuh"

#define RR_COLS 32                       // value columns of a CTA of the narrow form (the wide form takes 16); records pad v to this
#define RR_PREP_THREADS 128

struct RecurArgs {
    const void* q; long long ldq;          // [T, Hk * dk]   (activation dtype)
    const void* k; long long ldk;          // [T, Hk * dk]
    const void* v; long long ldv;          // [T, H * dv]
    const float* z; long long ldz;         // [T, H * dk] gate pre-activation without its bias ([T, H] with z_per_head)
    const float* z_bias;                   // [H * dk] or null ([H] with z_per_head)
    int z_per_head;                        // one gate per head and token instead of one per key channel
    const void* a_pre; long long lda;      // form 1: removal rate before the sigmoid [T, H * dk] (activation dtype)
    const float* a_bias;                   // form 1: [H * dk] or null
    const void* b_pre; long long ldb;      // form 2: write strength before the sigmoid [T, H]
    const float* rate;                     // gate 2: [H]
    float gate_param;                      // gate 0: 1 / tau;  gate 1: c
    float q_scale;                         // q is multiplied by this (after it was made a unit vector, if it is)
    int unit_qk;                           // q and k are made unit vectors: x / sqrt(sum x^2 + 1e-6)
    int gate;
    float* state;                          // [slots, H, dk, dv]
    float* out;                            // [T, H, dv]
    const int* cu_q; const int* entry_slot;
    int H, Hk, dk, dv, tile;
    float* prep;                           // [T, H, record] vectors prepared ahead (null: the walking kernel prepares them)
    int n_tokens;
    int rec_floats;                        // floats of a record made ahead: the vectors, then v of the head padded to RR_COLS columns
};

__device__ __forceinline__ void rr_cp_async16(void* dst, const void* src) {
    const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(d), "l"(src) : "memory");
}
__device__ __forceinline__ void rr_cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void rr_cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ float softplus_f(float x) { return fmaxf(x, 0.0f) + log1pf(expf(-fabsf(x))); }
__device__ __forceinline__ float sigmoid_f(float x) { return 1.0f / (1.0f + expf(-x)); }

// A token's record for one head: the vectors q, k, g - 1 (form 1 also u and a*u), each as SPLIT row slices of RP
// floats padded to RP + 4 (so that the slices of the lanes that share a column lie in different banks), then the
// write strength (form 2) and padding to 16 bytes.
template <int FORM, int SPLIT, int RP> struct RecurRecord {
    static constexpr int RPP = RP + 4;
    static constexpr int VEC = SPLIT * RPP;
    static constexpr int NARR = FORM == 1 ? 5 : 3;
    static constexpr int FLOATS = NARR * VEC + 4;
};

// One warp prepares token t of head h into `rec` (shared or global memory).
template <typename TA, int FORM, int SPLIT, int RP>
__device__ __forceinline__ void recur_prepare(const RecurArgs& A, size_t t, int h, int kvh, float rate, int lane, float* rec) {
    using R = RecurRecord<FORM, SPLIT, RP>;
    const int dk = A.dk;
    const TA* qr = (const TA*)A.q + t * A.ldq + (size_t)kvh * dk;
    const TA* kr = (const TA*)A.k + t * A.ldk + (size_t)kvh * dk;
    float qn = A.q_scale, kn = 1.0f, un = 1.0f;
    if (A.unit_qk || FORM == 1) {
        float sq = 0.0f, sk = 0.0f;
        for (int i = lane; i < dk; i += 32) {
            const float a = to_f32(qr[i]), b = to_f32(kr[i]);
            sq = fmaf(a, a, sq); sk = fmaf(b, b, sk);
        }
        sq = warp_sum(sq); sk = warp_sum(sk);
        if (A.unit_qk) { qn = A.q_scale / sqrtf(sq + 1e-6f); kn = 1.0f / sqrtf(sk + 1e-6f); }
        un = 1.0f / sqrtf(sk + 1e-6f);
    }
    for (int i = lane; i < SPLIT * RP; i += 32) {
        const int at = (i / RP) * R::RPP + (i % RP);
        float qv = 0.0f, kv = 0.0f, g = -1.0f, uv = 0.0f, av = 0.0f;
        if (i < dk) {
            qv = to_f32(qr[i]) * qn;
            const float kraw = to_f32(kr[i]);
            kv = kraw * kn;
            const size_t zi = A.z_per_head ? (size_t)h : (size_t)h * dk + i;
            float z = A.z[t * A.ldz + zi];
            if (A.z_bias) z += A.z_bias[zi];
            // the gate is kept as g - 1 = expm1(ln g): a gate close to 1 (a memory that lasts thousands of
            // tokens) then keeps the digits of 1 - g that rounding g itself to float would drop
            float lg;
            if (A.gate == 0) lg = -softplus_f(-z) * A.gate_param;
            else if (A.gate == 1) lg = -A.gate_param * sigmoid_f(z);
            else lg = -rate * softplus_f(z);
            g = expm1f(lg);
            if (FORM == 1) {
                float ap = to_f32(((const TA*)A.a_pre)[t * A.lda + (size_t)h * dk + i]);
                if (A.a_bias) ap += A.a_bias[(size_t)h * dk + i];
                uv = kraw * un;
                av = sigmoid_f(ap) * uv;
            }
        }
        rec[at] = qv; rec[R::VEC + at] = kv; rec[2 * R::VEC + at] = g;
        if (FORM == 1) { rec[3 * R::VEC + at] = uv; rec[4 * R::VEC + at] = av; }
    }
    if (lane < 4) {
        float b = 0.0f;
        if (FORM == 2 && lane == 0) b = sigmoid_f(to_f32(((const TA*)A.b_pre)[t * A.ldb + h]));
        rec[R::NARR * R::VEC + lane] = b;
    }
}

// The preparation ahead: one warp per (token, head) of the step.
template <typename TA, int FORM, int SPLIT, int RP>
__global__ void __launch_bounds__(RR_PREP_THREADS)
recurrence_prepare_kernel(const RecurArgs A) {
    pdl_trigger();
    const long long w = (long long)blockIdx.x * (RR_PREP_THREADS / 32) + (threadIdx.x >> 5);
    const bool live = w < (long long)A.n_tokens * A.H;
    const int h = live ? (int)(w % A.H) : 0;
    const float rate = (live && A.gate == 2) ? expf(A.rate[h]) : 0.0f;
    pdl_wait();
    if (!live) return;
    const size_t t = (size_t)(w / A.H);
    const int lane = threadIdx.x & 31;
    float* rec = A.prep + (size_t)w * A.rec_floats;
    recur_prepare<TA, FORM, SPLIT, RP>(A, t, h, h / (A.H / A.Hk), rate, lane, rec);
    // the head's values as floats, padded with zeros to whole blocks of RR_COLS columns
    const TA* vr = (const TA*)A.v + t * A.ldv + (size_t)h * A.dv;
    float* vd = rec + RecurRecord<FORM, SPLIT, RP>::FLOATS;
    for (int i = lane; i < A.rec_floats - RecurRecord<FORM, SPLIT, RP>::FLOATS; i += 32) vd[i] = i < A.dv ? to_f32(vr[i]) : 0.0f;
}

__device__ __forceinline__ float sum4(const float4 v) { return (v.x + v.y) + (v.z + v.w); }
template <int SPLIT> __device__ __forceinline__ float split_sum(float v) {          // over the lanes that share a column
#pragma unroll
    for (int o = 1; o < SPLIT; o <<= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}

template <typename TA, int FORM, int SPLIT, int RP, bool AHEAD, int COLS>
__global__ void __launch_bounds__(COLS * SPLIT)
recurrence_kernel(const RecurArgs A) {
    constexpr int RR_THREADS = COLS * SPLIT;
    using R = RecurRecord<FORM, SPLIT, RP>;
    constexpr int RPP = R::RPP, VEC = R::VEC, REC = R::FLOATS;
    extern __shared__ __align__(16) float sm[];
    pdl_trigger();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int h = blockIdx.y, e = blockIdx.z;
    const int c0 = blockIdx.x * COLS;
    const int kvh = h / (A.H / A.Hk);
    const int dk = A.dk, dv = A.dv, TT = A.tile;
    float* recs = sm;                                  // [TT][REC]
    float* vs = sm + TT * REC;                         // [TT][COLS]
    const float rate = (!AHEAD && A.gate == 2) ? expf(A.rate[h]) : 0.0f;     // weights: read before the wait
    pdl_wait();
    const int s0 = A.cu_q[e], n = A.cu_q[e + 1] - s0;
    const int slot = A.entry_slot[e];
    const int cl = warp * (32 / SPLIT) + lane / SPLIT;       // column of this thread inside the CTA's block
    const int r = lane % SPLIT;
    const int c = c0 + cl;
    float* S = A.state + ((size_t)slot * A.H + h) * dk * dv;
    float s[RP];
#pragma unroll
    for (int ii = 0; ii < RP; ++ii) {
        const int i = r * RP + ii;
        s[ii] = (i < dk && c < dv) ? S[(size_t)i * dv + c] : 0.0f;
    }
    const TA* v = (const TA*)A.v;
    // Records made ahead arrive by asynchronous copies, the next tile's while this one is walked (two buffers).
    constexpr int R4 = REC / 4, V4 = COLS / 4;
    const int stride = TT * (REC + COLS);           // floats of one buffer: [TT][REC] then [TT][COLS]
    auto fetch = [&](int buf, int base) {
        const int nt = min(TT, n - base);
        float* dst = sm + buf * stride;
        for (int idx = threadIdx.x; idx < nt * (R4 + V4); idx += RR_THREADS) {
            const int tt = idx / (R4 + V4), w4 = idx - tt * (R4 + V4);
            const float* src = A.prep + ((size_t)(s0 + base + tt) * A.H + h) * A.rec_floats;
            if (w4 < R4) rr_cp_async16(dst + tt * REC + 4 * w4, src + 4 * w4);
            else rr_cp_async16(dst + TT * REC + tt * COLS + 4 * (w4 - R4), src + REC + c0 + 4 * (w4 - R4));
        }
        rr_cp_async_commit();
    };
    float* opart = sm + (AHEAD ? 2 : 1) * stride;      // [TT][COLS][SPLIT] parts of the read-out
    if (AHEAD && n > 0) fetch(0, 0);
    for (int base = 0, it = 0; base < n; base += TT, ++it) {
        const int nt = min(TT, n - base);
        if (AHEAD) {
            if (base + TT < n) { fetch((it + 1) & 1, base + TT); rr_cp_async_wait<1>(); }
            else rr_cp_async_wait<0>();
            recs = sm + (it & 1) * stride;
            vs = recs + TT * REC;
        } else {
            __syncthreads();                           // the tile before has been read by everybody
            for (int tt = warp; tt < nt; tt += RR_THREADS / 32) {
                const size_t t = (size_t)(s0 + base + tt);
                recur_prepare<TA, FORM, SPLIT, RP>(A, t, h, kvh, rate, lane, recs + tt * REC);
                const int cc = c0 + lane;              // a lane per column
                if (lane < COLS) vs[tt * COLS + lane] = cc < dv ? to_f32(v[t * A.ldv + (size_t)h * dv + cc]) : 0.0f;
            }
        }
        __syncthreads();
        // ---- walk the tile
        for (int tt = 0; tt < nt; ++tt) {
            const float* rec = recs + tt * REC + r * RPP;
            const float4* q4 = (const float4*)rec;
            const float4* k4 = (const float4*)(rec + VEC);
            const float4* g4 = (const float4*)(rec + 2 * VEC);
            const float vc = vs[tt * COLS + cl];
            float4 o4 = make_float4(0.0f, 0.0f, 0.0f, 0.0f);      // four chains, joined in a fixed order
            if (FORM == 0) {
#pragma unroll
                for (int j = 0; j < RP / 4; ++j) {
                    const float4 qq = q4[j], kk = k4[j], gg = g4[j];
                    s[4 * j + 0] = fmaf(gg.x, s[4 * j + 0], fmaf(kk.x, vc, s[4 * j + 0])); o4.x = fmaf(s[4 * j + 0], qq.x, o4.x);
                    s[4 * j + 1] = fmaf(gg.y, s[4 * j + 1], fmaf(kk.y, vc, s[4 * j + 1])); o4.y = fmaf(s[4 * j + 1], qq.y, o4.y);
                    s[4 * j + 2] = fmaf(gg.z, s[4 * j + 2], fmaf(kk.z, vc, s[4 * j + 2])); o4.z = fmaf(s[4 * j + 2], qq.z, o4.z);
                    s[4 * j + 3] = fmaf(gg.w, s[4 * j + 3], fmaf(kk.w, vc, s[4 * j + 3])); o4.w = fmaf(s[4 * j + 3], qq.w, o4.w);
                }
            } else if (FORM == 1) {
                const float4* u4 = (const float4*)(rec + 3 * VEC);
                const float4* a4 = (const float4*)(rec + 4 * VEC);
                float4 d4 = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll
                for (int j = 0; j < RP / 4; ++j) {
                    const float4 uu = u4[j];
                    d4.x = fmaf(uu.x, s[4 * j + 0], d4.x); d4.y = fmaf(uu.y, s[4 * j + 1], d4.y);
                    d4.z = fmaf(uu.z, s[4 * j + 2], d4.z); d4.w = fmaf(uu.w, s[4 * j + 3], d4.w);
                }
                const float dot = split_sum<SPLIT>(sum4(d4));
#pragma unroll
                for (int j = 0; j < RP / 4; ++j) {
                    const float4 qq = q4[j], kk = k4[j], gg = g4[j], aa = a4[j];
                    s[4 * j + 0] = fmaf(gg.x, s[4 * j + 0], s[4 * j + 0] + fmaf(-aa.x, dot, kk.x * vc)); o4.x = fmaf(s[4 * j + 0], qq.x, o4.x);
                    s[4 * j + 1] = fmaf(gg.y, s[4 * j + 1], s[4 * j + 1] + fmaf(-aa.y, dot, kk.y * vc)); o4.y = fmaf(s[4 * j + 1], qq.y, o4.y);
                    s[4 * j + 2] = fmaf(gg.z, s[4 * j + 2], s[4 * j + 2] + fmaf(-aa.z, dot, kk.z * vc)); o4.z = fmaf(s[4 * j + 2], qq.z, o4.z);
                    s[4 * j + 3] = fmaf(gg.w, s[4 * j + 3], s[4 * j + 3] + fmaf(-aa.w, dot, kk.w * vc)); o4.w = fmaf(s[4 * j + 3], qq.w, o4.w);
                }
            } else {
                float4 d4 = make_float4(0.0f, 0.0f, 0.0f, 0.0f);
#pragma unroll
                for (int j = 0; j < RP / 4; ++j) {
                    const float4 kk = k4[j], gg = g4[j];
                    s[4 * j + 0] = fmaf(gg.x, s[4 * j + 0], s[4 * j + 0]); d4.x = fmaf(kk.x, s[4 * j + 0], d4.x);
                    s[4 * j + 1] = fmaf(gg.y, s[4 * j + 1], s[4 * j + 1]); d4.y = fmaf(kk.y, s[4 * j + 1], d4.y);
                    s[4 * j + 2] = fmaf(gg.z, s[4 * j + 2], s[4 * j + 2]); d4.z = fmaf(kk.z, s[4 * j + 2], d4.z);
                    s[4 * j + 3] = fmaf(gg.w, s[4 * j + 3], s[4 * j + 3]); d4.w = fmaf(kk.w, s[4 * j + 3], d4.w);
                }
                const float dot = split_sum<SPLIT>(sum4(d4));
                const float dl = recs[tt * REC + R::NARR * VEC] * (vc - dot);
#pragma unroll
                for (int j = 0; j < RP / 4; ++j) {
                    const float4 qq = q4[j], kk = k4[j];
                    s[4 * j + 0] = fmaf(kk.x, dl, s[4 * j + 0]); o4.x = fmaf(s[4 * j + 0], qq.x, o4.x);
                    s[4 * j + 1] = fmaf(kk.y, dl, s[4 * j + 1]); o4.y = fmaf(s[4 * j + 1], qq.y, o4.y);
                    s[4 * j + 2] = fmaf(kk.z, dl, s[4 * j + 2]); o4.z = fmaf(s[4 * j + 2], qq.z, o4.z);
                    s[4 * j + 3] = fmaf(kk.w, dl, s[4 * j + 3]); o4.w = fmaf(s[4 * j + 3], qq.w, o4.w);
                }
            }
            // the read-out is not part of the chain from token to token: the lanes leave their parts, and the
            // tile's sums are formed afterwards, all at once
            opart[(tt * COLS + cl) * SPLIT + r] = sum4(o4);
        }
        __syncthreads();                               // the parts are written; and (AHEAD) this buffer is refilled by the fetch after next
        for (int idx = threadIdx.x; idx < nt * COLS; idx += RR_THREADS) {
            const float* part = opart + idx * SPLIT;
            float o = part[0];
#pragma unroll
            for (int i = 1; i < SPLIT; ++i) o += part[i];
            const int tt = idx / COLS, cc = c0 + idx % COLS;
            if (cc < dv) A.out[((size_t)(s0 + base + tt) * A.H + h) * dv + cc] = o;
        }
    }
#pragma unroll
    for (int ii = 0; ii < RP; ++ii) {
        const int i = r * RP + ii;
        if (i < dk && c < dv) S[(size_t)i * dv + c] = s[ii];
    }
}

// Lanes per column and rows per lane for a key size: (4, 8..64) is the narrow form; the wide form (long bfloat16
// portions) is (8, 8) up to 64 key channels, (16, 8) up to 128, (16, 16) up to 256.
static void recurrence_shape(int dk, bool wide, int* split, int* rp) {
    if (wide && dk > 32) {
        *split = dk <= 64 ? 8 : 16;
        *rp = dk <= 128 ? 8 : 16;
        return;
    }
    const int need = rb_ceil_div(dk, 4);
    *split = 4;
    *rp = need <= 8 ? 8 : need <= 16 ? 16 : need <= 32 ? 32 : 64;
}

template <typename TA, int FORM, int SPLIT, int RP, bool AHEAD>
static int recurrence_launch(const RecurArgs& A, int n_entries, cudaStream_t st) {
    using R = RecurRecord<FORM, SPLIT, RP>;
    // the wide form: 16 columns a CTA, so that the CTAs of one long portion spread over twice as many SMs
    constexpr int COLS = SPLIT > 4 ? 16 : RR_COLS;
    RecurArgs a = A;
    a.tile = (R::FLOATS + COLS) * 16 * sizeof(float) * (AHEAD ? 2 : 1) > 160 * 1024 || RP >= 64 ? 8 : 16;
    const size_t smem = (size_t)a.tile * ((R::FLOATS + COLS) * (AHEAD ? 2 : 1) + COLS * SPLIT) * sizeof(float);
    dim3 grid(rb_ceil_div(a.dv, COLS), a.H, n_entries);
    static bool done = false;                          // two buffers may pass the default limit of dynamic shared memory
    if (!done && smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(recurrence_kernel<TA, FORM, SPLIT, RP, AHEAD, COLS>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        done = true;
    }
    if (AHEAD) {
        a.rec_floats = R::FLOATS + rb_ceil_div(a.dv, RR_COLS) * RR_COLS;
        const long long warps = (long long)a.n_tokens * a.H;
        int rc = rb_launch(recurrence_prepare_kernel<TA, FORM, SPLIT, RP>, dim3(rb_ceil_div(warps, RR_PREP_THREADS / 32)),
                           dim3(RR_PREP_THREADS), 0, st, a);
        if (rc) return rc;
    } else {
        a.prep = nullptr;
    }
    return rb_launch(recurrence_kernel<TA, FORM, SPLIT, RP, AHEAD, COLS>, grid, dim3(COLS * SPLIT), smem, st, a);
}

template <typename TA, int FORM, bool WIDE_OK>
static int recurrence_dispatch(const RecurArgs& A, int n_entries, int max_q_len, cudaStream_t st) {
    int tile_probe_split, rp;
    recurrence_shape(A.dk, false, &tile_probe_split, &rp);
    const bool ahead = A.prep != nullptr && max_q_len > (rp >= 64 ? 8 : 16);
    int split;
    recurrence_shape(A.dk, WIDE_OK && ahead, &split, &rp);
    if (ahead) {
        if (WIDE_OK && split == 8) return recurrence_launch<TA, FORM, 8, 8, true>(A, n_entries, st);
        if (WIDE_OK && split == 16 && rp == 8) return recurrence_launch<TA, FORM, 16, 8, true>(A, n_entries, st);
        if (WIDE_OK && split == 16) return recurrence_launch<TA, FORM, 16, 16, true>(A, n_entries, st);
        if (rp == 8) return recurrence_launch<TA, FORM, 4, 8, true>(A, n_entries, st);
        if (rp == 16) return recurrence_launch<TA, FORM, 4, 16, true>(A, n_entries, st);
        if (rp == 32) return recurrence_launch<TA, FORM, 4, 32, true>(A, n_entries, st);
        return recurrence_launch<TA, FORM, 4, 64, true>(A, n_entries, st);
    }
    if (rp == 8) return recurrence_launch<TA, FORM, 4, 8, false>(A, n_entries, st);
    if (rp == 16) return recurrence_launch<TA, FORM, 4, 16, false>(A, n_entries, st);
    if (rp == 32) return recurrence_launch<TA, FORM, 4, 32, false>(A, n_entries, st);
    return recurrence_launch<TA, FORM, 4, 64, false>(A, n_entries, st);
}

// Floats of scratch per (token, head) that the preparation ahead needs (the largest over the forms of the kernel that
// this key size can take).
extern "C" int rb_recurrence_record_floats(int form, int dk, int dv) {
    int best = 0;
    for (int wide = 0; wide < 2; ++wide) {
        int split, rp;
        recurrence_shape(dk, wide != 0, &split, &rp);
        const int f = (form == 1 ? 5 : 3) * split * (rp + 4) + 4;
        best = f > best ? f : best;
    }
    return best + rb_ceil_div(dv, RR_COLS) * RR_COLS;
}
// Tokens of a portion up to which the walking kernel prepares its vectors itself.
extern "C" int rb_recurrence_tile(int dk) { return rb_ceil_div(dk, 4) > 32 ? 8 : 16; }

// form: 0, 1, 2 as above.  All row strides in elements.  state [slots, H, dk, dv] float; out [T, H, dv] float.
// prep: scratch of n_tokens * H * rb_recurrence_record_floats() floats, or null; it is used when max_q_len (the
// step's longest portion) exceeds one tile.
extern "C" int rb_recurrence(int form, int gate, int dtype,
                             const void* q, long long ldq, const void* k, long long ldk, const void* v, long long ldv,
                             const float* z, long long ldz, const float* z_bias, int z_per_head,
                             const void* a_pre, long long lda, const float* a_bias,
                             const void* b_pre, long long ldb, const float* rate,
                             float gate_param, float q_scale, int unit_qk,
                             float* state, float* out, const int* cu_q, const int* entry_slot,
                             int n_entries, int H, int Hk, int dk, int dv, float* prep, int n_tokens, int max_q_len, void* stream) {
    if (n_entries <= 0) return 0;
    if (H <= 0 || Hk <= 0 || H % Hk) RB_REFUSE("recurrence: %d heads over %d key heads", H, Hk);
    if (dk <= 0 || dk > 256 || dv <= 0) RB_REFUSE("recurrence: key size %d (1..256), value size %d", dk, dv);
    if (form < 0 || form > 2 || gate < 0 || gate > 2) RB_REFUSE("recurrence: form %d, gate %d", form, gate);
    if (form == 1 && !a_pre) RB_REFUSE("recurrence: the delta form on the old state needs removal rates");
    if (form == 2 && !b_pre) RB_REFUSE("recurrence: the gated delta form needs write strengths");
    if (gate == 2 && !rate) RB_REFUSE("recurrence: gate 2 needs a rate per head");
    if (n_entries > 65535 || H > 65535) RB_REFUSE("recurrence: %d requests, %d heads exceed the grid", n_entries, H);
    RecurArgs A;
    A.q = q; A.ldq = ldq; A.k = k; A.ldk = ldk; A.v = v; A.ldv = ldv; A.z = z; A.ldz = ldz; A.z_bias = z_bias; A.z_per_head = z_per_head;
    A.a_pre = a_pre; A.lda = lda; A.a_bias = a_bias; A.b_pre = b_pre; A.ldb = ldb; A.rate = rate;
    A.gate_param = gate_param; A.q_scale = q_scale; A.unit_qk = unit_qk; A.gate = gate;
    A.state = state; A.out = out; A.cu_q = cu_q; A.entry_slot = entry_slot;
    A.H = H; A.Hk = Hk; A.dk = dk; A.dv = dv; A.tile = 16; A.prep = prep; A.n_tokens = n_tokens; A.rec_floats = 0;
    cudaStream_t st = (cudaStream_t)stream;
#define RB_RECUR(TA, WIDE) \
    do { if (form == 0) return recurrence_dispatch<TA, 0, WIDE>(A, n_entries, max_q_len, st); \
         if (form == 1) return recurrence_dispatch<TA, 1, WIDE>(A, n_entries, max_q_len, st); \
         return recurrence_dispatch<TA, 2, WIDE>(A, n_entries, max_q_len, st); } while (0)
    if (dtype == RB_F32) RB_RECUR(float, false);
    if (dtype == RB_BF16) RB_RECUR(bf16, true);
#undef RB_RECUR
    RB_REFUSE("recurrence: dtype %d", dtype);
}
