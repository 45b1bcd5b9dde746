// Flash attention over the paged cache for the bfloat16 path: one kernel body in two
// shapes.  Keys and values are brought page by page into shared memory with cp.async
// (16-byte copies, zero fill for what lies outside the request), scores and the
// probability-weighted values go through mma.sync m16n8k16 (bf16 in, float out), the
// softmax is online and in float (exp2 of scores pre-multiplied by scale*log2 e).
//
//  * PREFILL (entries that bring more than one token): a CTA owns 64 rows = 64/Gc tokens
//    x Gc query heads of one kv head (grouped heads share every K/V tile they read), each
//    warp 16 rows, all warps walk the same 64-key tiles from the request's pages -
//    including the pages that EARLIER steps wrote, which the reference's prefill kernel
//    cannot read (it attends to the fresh K/V of one call only,
//    bin/reinfer/src/sched_loop.rs:188-195; crates/cuda/src/fmha.rs:711-729).
//  * DECODE (one token): the Gc query heads of a kv head are the rows of ONE 16-row tile;
//    the request's keys are split across CTAs (grid.z) and inside a CTA across the four
//    warps (16 keys of each 64-key tile per warp); warps merge in shared memory, CTAs
//    through a scratch buffer and a small merge kernel, in fixed order.  (The reference
//    runs one CTA per query head over the whole context and re-reads K/V per head,
//    crates/cuda/kernels/decode_flash_kernels.cu:167-369.)
//
// Two optional extras serve attention that is local to chunks of positions and has no rotation: a chunk mask (a row
// sees only the keys from the start of its own chunk of `chunk` positions, counted from position 0) and a penalty on
// distance per query head, score -= r1[h] ln(1 + r2[h] (i - j)), added in the exponent's base-2 domain as
// r1 log2(1 + r2 (i - j)); and a factor on the output.  Two more serve attention with a learned bias by distance and
// value heads of their own size: a float table bias[head][min(i - j, rows - 1)] that is added to the scaled score
// (the last column stands for every greater distance), and dv != d (a page is then [K: KH x page x d | V: KH x page x
// dv]; the tiles are as wide as the larger of the two, the narrower zero-filled).  Four more: scores squashed to
// cap * tanh(score / cap); a sink per query head that joins the softmax's denominator as exp(sink[h]) and brings no
// value (added once: by the CTA where the keys are not split, else by the merge); values that are the first dv columns
// of the key rows (a page then holds keys only); and a gate, out *= sigmoid(gate[t][h * dv + i]), on float rows with a
// stride of their own.  Without them the kernels are what they were.
//
// Head sizes: the template is instantiated for 32, 64, 128 and 256; a head size that is a
// multiple of 8 below the next instance is zero-padded in shared memory.  The prefill kernel has one more shape for a
// key head of 256 that holds values of at most 192 columns (latent attention): tiles of 32 keys, three CTAs a SM.
#include "common.cuh"

#define FA_WARPS 4
#define FA_THREADS (FA_WARPS * 32)
#define FA_BN 64                       // keys per tile
#define FA_BM 64                       // rows per prefill CTA

struct FaArgs {
    const bf16* q;                     // [T, QH, d]
    const bf16* cache;                 // one layer: [page][2][KH][page_size][d]
    const int* block_table;            // [entries, max_pages]
    const int* cu_q;                   // [entries + 1]
    const int* kv_len;                 // [entries] length of the request after this step
    bf16* out;                         // [T, QH, d]
    float* part_o;                     // decode: [tokens, QH, splits, d] normalised partial outputs
    float* part_lse;                   // decode: [tokens, QH, splits] log2 of the partial softmax sums
    int QH, KH, d, page_size, max_pages, window;
    int page_shift;                    // log2(page_size), or -1 if it is no power of two
    int Gc, chunks;                    // query heads per row tile (divides QH/KH, <= 16), tiles per kv head
    int first_entry, n_entries;        // entries this launch covers: [first_entry, first_entry + n_entries)
    int n_splits;
    float scale_log2;
    int chunk;                         // > 0: keys before floor(pos / chunk) * chunk are not seen
    const float* r1;                   // [QH] distance penalty (null: none)
    const float* r2;
    float out_scale;
    int dv;                            // the value heads' size (= d unless the layer says otherwise)
    const float* bias;                 // [QH, bias_rows] added to the scaled scores by distance (null: none)
    int bias_rows;
    float cap_log2, scale_over_cap;    // soft cap: score <- cap tanh(score / cap), here cap * log2 e and scale / cap (0: none)
    const float* sink;                 // [QH] one more term exp(sink[h]) in the denominator (null: none)
    int v_in_k;                        // != 0: the values are the first dv columns of the key rows; pages hold keys only
    const float* gate;                 // out *= sigmoid(gate[t * gate_stride + h * dv + i]) (null: none)
    long long gate_stride;
};

__device__ __forceinline__ float fa_sigmoid(float z) { return 1.0f / (1.0f + expf(-z)); }
// 2^x for x <= 0 or -inf by the special-function unit alone (exp2f wraps range handling around the same instruction;
// results below 2^-126 are flushed to zero, which P, rounded to bfloat16, and the rescaling factors do not feel)
__device__ __forceinline__ float fa_ex2(float x) {
    float y;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(y) : "f"(x));
    return y;
}

// ---------------------------------------------------------------- small PTX wrappers
__device__ __forceinline__ void cp_async16(void* dst, const void* src, int src_bytes) {
    const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
template <int N> __device__ __forceinline__ void cp_async_wait() { asm volatile("cp.async.wait_group %0;" ::"n"(N) : "memory"); }

__device__ __forceinline__ void ldsm_x4(uint32_t (&r)[4], const void* p) {
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void ldsm_x4_trans(uint32_t (&r)[4], const void* p) {
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void mma_bf16(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3])
                 : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 v = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&v);
}

template <int D, int BN = FA_BN> struct FaSmem {
    static constexpr int STRIDE = D * 2 + 16;                 // bytes per row: 16 bytes of padding keep ldmatrix conflict-free
    static constexpr int TILE = BN * STRIDE;                  // one K or V tile (BN keys)
    static constexpr int STAGE = 2 * TILE;                    // keys and values
    static constexpr int STAGE_VK = TILE;                     // values inside the keys: the key tile serves both products
};
template <int D, bool VK, int BN = FA_BN> __host__ __device__ constexpr int fa_stage() { return VK ? FaSmem<D, BN>::STAGE_VK : FaSmem<D, BN>::STAGE; }

// Copy keys [k0, k0+64) of kv head `kh` (K and V) of the request whose block-table row is `bt`
// into one stage.  Rows at or beyond `kv_end`, rows in pages that were given back (id < 0) and
// the padding dims d..D are zero-filled, so nothing that is not the request's own data is read.
// A thread always copies the same 16-byte column of rows r0, r0 + RPI, ...; with a page size that
// is a power of two (page_shift >= 0) the page of a row costs a shift and a mask.  VK: the values are the first dv
// columns of the key rows and the stage holds the key tile only.
template <int D, bool VK, int BN = FA_BN>
__device__ __forceinline__ void fa_load_tile(unsigned char* stage, const FaArgs& a, const int* bt, int kh, int k0, int kv_end) {
    constexpr int CPR = D / 8;                                // 16-byte chunks per row
    constexpr int RPI = FA_THREADS / CPR;                     // rows per pass over the tile
    static_assert(FA_THREADS % CPR == 0 && BN % RPI == 0, "tile shape");
    const int c = threadIdx.x % CPR, r0 = threadIdx.x / CPR;
    const bool kcol_ok = c * 8 < a.d, vcol_ok = c * 8 < a.dv;
    const size_t head_stride = (size_t)a.page_size * a.d, vhead_stride = VK ? head_stride : (size_t)a.page_size * a.dv;
    const size_t page_stride = VK ? (size_t)a.KH * head_stride : (size_t)a.KH * (head_stride + vhead_stride);
    const int v_row = VK ? a.d : a.dv;
    const bf16* kbase = a.cache + (size_t)kh * head_stride + c * 8;
    const bf16* vbase = a.cache + (VK ? 0 : (size_t)a.KH * head_stride) + (size_t)kh * vhead_stride + c * 8;
    unsigned char* dst0 = stage + r0 * FaSmem<D>::STRIDE + c * 16;
#pragma unroll
    for (int i = 0; i < BN / RPI; ++i) {
        const int key = k0 + r0 + i * RPI;
        const bf16* ksrc = a.cache;
        const bf16* vsrc = a.cache;
        int kbytes = 0, vbytes = 0;
        if (key < kv_end) {
            int pi, off;
            if (a.page_shift >= 0) { pi = key >> a.page_shift; off = key & (a.page_size - 1); }
            else { pi = key / a.page_size; off = key - pi * a.page_size; }
            const int page = pi < a.max_pages ? bt[pi] : -1;
            if (page >= 0) {
                if (kcol_ok) { ksrc = kbase + (size_t)page * page_stride + (size_t)off * a.d; kbytes = 16; }
                if (vcol_ok) { vsrc = vbase + (size_t)page * page_stride + (size_t)off * v_row; vbytes = 16; }
            }
        }
        unsigned char* dst = dst0 + i * RPI * FaSmem<D>::STRIDE;
        cp_async16(dst, ksrc, kbytes);
        if (!VK) cp_async16(dst + FaSmem<D, BN>::TILE, vsrc, vbytes);
    }
}

// One 64-key tile for one warp: scores of its 16 rows against NT n-tiles of 8 keys starting at
// key `koff` of the tile, online softmax, and the P V update.
//   pos0/pos1, lo0/lo1: last and first visible key of row lane/4 and row lane/4 + 8.
template <int D, int NT, int DO = D>
__device__ __forceinline__ void fa_tile(const unsigned char* sQ, const unsigned char* sK, const unsigned char* sV,
                                        int koff, int k0_abs, int pos0, int pos1, int lo0, int lo1, float scale_log2,
                                        float (&o)[DO / 8][4], float (&m)[2], float (&l)[2],
                                        bool pen = false, float pa0 = 0.0f, float pb0 = 0.0f, float pa1 = 0.0f, float pb1 = 0.0f,
                                        const float* bias0 = nullptr, const float* bias1 = nullptr, int bias_stride = 0, int bias_last = 0,
                                        float cap_log2 = 0.0f, float scale_over_cap = 0.0f, int dv_cols = D) {
    constexpr int STRIDE = FaSmem<D>::STRIDE;
    const int lane = threadIdx.x & 31;
    float s[NT][4];
#pragma unroll
    for (int j = 0; j < NT; ++j) { s[j][0] = s[j][1] = s[j][2] = s[j][3] = 0.0f; }
#pragma unroll
    for (int ks = 0; ks < D / 16; ++ks) {
        uint32_t qa[4];
        ldsm_x4(qa, sQ + ((lane & 7) + 8 * ((lane >> 3) & 1)) * STRIDE + (ks * 16 + 8 * (lane >> 4)) * 2);
#pragma unroll
        for (int jp = 0; jp < NT / 2; ++jp) {
            uint32_t kb[4];
            ldsm_x4(kb, sK + (koff + jp * 16 + (lane & 7) + 8 * (lane >> 4)) * STRIDE + (ks * 16 + 8 * ((lane >> 3) & 1)) * 2);
            mma_bf16(s[2 * jp], qa, kb[0], kb[1]);
            mma_bf16(s[2 * jp + 1], qa, kb[2], kb[3]);
        }
    }
    // scale, mask, row maxima
    float mx0 = -INFINITY, mx1 = -INFINITY;
#pragma unroll
    for (int j = 0; j < NT; ++j) {
        const int key = k0_abs + koff + j * 8 + 2 * (lane & 3);
        float v0 = s[j][0] * scale_log2, v1 = s[j][1] * scale_log2, v2 = s[j][2] * scale_log2, v3 = s[j][3] * scale_log2;
        if (cap_log2 > 0.0f) {                                 // the soft cap, in the exponent's base-2 domain
            v0 = cap_log2 * tanhf(s[j][0] * scale_over_cap); v1 = cap_log2 * tanhf(s[j][1] * scale_over_cap);
            v2 = cap_log2 * tanhf(s[j][2] * scale_over_cap); v3 = cap_log2 * tanhf(s[j][3] * scale_over_cap);
        }
        if (pen) {                                             // the distance penalty (masked places are replaced below)
            v0 = fmaf(-pa0, __log2f(fmaf(pb0, (float)(pos0 - key), 1.0f)), v0);
            v1 = fmaf(-pa0, __log2f(fmaf(pb0, (float)(pos0 - key - 1), 1.0f)), v1);
            v2 = fmaf(-pa1, __log2f(fmaf(pb1, (float)(pos1 - key), 1.0f)), v2);
            v3 = fmaf(-pa1, __log2f(fmaf(pb1, (float)(pos1 - key - 1), 1.0f)), v3);
        }
        if (bias0) {                                           // the learned bias by distance, in the exponent's base-2 domain
            constexpr float LOG2E = 1.4426950408889634f;
            v0 = fmaf(bias0[(size_t)min(max(pos0 - key, 0), bias_last) * bias_stride], LOG2E, v0);
            v1 = fmaf(bias0[(size_t)min(max(pos0 - key - 1, 0), bias_last) * bias_stride], LOG2E, v1);
        }
        if (bias1) {
            constexpr float LOG2E = 1.4426950408889634f;
            v2 = fmaf(bias1[(size_t)min(max(pos1 - key, 0), bias_last) * bias_stride], LOG2E, v2);
            v3 = fmaf(bias1[(size_t)min(max(pos1 - key - 1, 0), bias_last) * bias_stride], LOG2E, v3);
        }
        s[j][0] = (key >= lo0 && key <= pos0) ? v0 : -INFINITY;
        s[j][1] = (key + 1 >= lo0 && key + 1 <= pos0) ? v1 : -INFINITY;
        s[j][2] = (key >= lo1 && key <= pos1) ? v2 : -INFINITY;
        s[j][3] = (key + 1 >= lo1 && key + 1 <= pos1) ? v3 : -INFINITY;
        mx0 = fmaxf(mx0, fmaxf(s[j][0], s[j][1]));
        mx1 = fmaxf(mx1, fmaxf(s[j][2], s[j][3]));
    }
    mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 1)); mx0 = fmaxf(mx0, __shfl_xor_sync(0xffffffffu, mx0, 2));
    mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 1)); mx1 = fmaxf(mx1, __shfl_xor_sync(0xffffffffu, mx1, 2));
    const float mn0 = fmaxf(m[0], mx0), mn1 = fmaxf(m[1], mx1);
    const float base0 = mn0 == -INFINITY ? 0.0f : mn0, base1 = mn1 == -INFINITY ? 0.0f : mn1;   // a row that saw no key yet
    const float c0 = fa_ex2(m[0] - base0), c1 = fa_ex2(m[1] - base1);
    m[0] = mn0; m[1] = mn1;
    float sum0 = 0.0f, sum1 = 0.0f;
    uint32_t p[NT][2];
#pragma unroll
    for (int j = 0; j < NT; ++j) {
        const float e0 = fa_ex2(s[j][0] - base0), e1 = fa_ex2(s[j][1] - base0);
        const float e2 = fa_ex2(s[j][2] - base1), e3 = fa_ex2(s[j][3] - base1);
        sum0 += e0 + e1; sum1 += e2 + e3;
        p[j][0] = pack_bf16(e0, e1);
        p[j][1] = pack_bf16(e2, e3);
    }
    l[0] = l[0] * c0 + sum0;                                   // per-thread partial sums; joined at the end
    l[1] = l[1] * c1 + sum1;
    // (a tile that raised no row's maximum leaves every factor at one: the whole warp skips the pass over its sums)
    if (__any_sync(0xffffffffu, c0 != 1.0f || c1 != 1.0f)) {
#pragma unroll
        for (int j = 0; j < DO / 8; ++j) { o[j][0] *= c0; o[j][1] *= c0; o[j][2] *= c1; o[j][3] *= c1; }
    }
    // O += P V
#pragma unroll
    for (int kk = 0; kk < NT / 2; ++kk) {
        const uint32_t pa[4] = {p[2 * kk][0], p[2 * kk][1], p[2 * kk + 1][0], p[2 * kk + 1][1]};
#pragma unroll
        for (int dp = 0; dp < DO / 16; ++dp) {
            if (dp * 16 >= dv_cols) continue;                  // columns beyond the value heads' size stay zero (the same for the whole CTA)
            uint32_t vb[4];
            ldsm_x4_trans(vb, sV + (koff + kk * 16 + (lane & 7) + 8 * ((lane >> 3) & 1)) * STRIDE + (dp * 16 + 8 * (lane >> 4)) * 2);
            mma_bf16(o[2 * dp], pa, vb[0], vb[1]);
            mma_bf16(o[2 * dp + 1], pa, vb[2], vb[3]);
        }
    }
}

// Load `rows` rows of Q (row r = token q_tok0 + r / Gc, head head0 + r % Gc) into shared memory, zero beyond.
template <int D>
__device__ __forceinline__ void fa_load_q(unsigned char* sQ, const FaArgs& a, int tok_base, int n_tok, int head0, int n_rows_smem) {
    constexpr int CPR = D / 8;
    for (int i = threadIdx.x; i < n_rows_smem * CPR; i += FA_THREADS) {
        const int row = i / CPR, c = i % CPR;
        const int ti = row / a.Gc, g = row % a.Gc;
        uint4 v = make_uint4(0, 0, 0, 0);
        if (ti < n_tok && c * 8 < a.d)
            v = *reinterpret_cast<const uint4*>(a.q + ((size_t)(tok_base + ti) * a.QH + head0 + g) * a.d + c * 8);
        *reinterpret_cast<uint4*>(sQ + row * FaSmem<D>::STRIDE + c * 16) = v;
    }
}

// ------------------------------------------------------------------------ prefill
// BN: keys per tile; DO: columns of the sums a warp keeps (>= the value heads' size); MINB: CTAs a SM that the
// registers are to leave room for.  A key head of 256 that holds its values takes tiles of 32 keys and 192 columns:
// three CTAs a SM where tiles of 64 keys and 256 columns leave two.
template <int D, bool VK, int BN = FA_BN, int DO = D, int MINB = 1>
__global__ void __launch_bounds__(FA_THREADS, MINB)
fa_prefill_kernel(const FaArgs a) {
    constexpr int NST = 2;
    constexpr int STAGE = fa_stage<D, VK, BN>();
    extern __shared__ __align__(16) unsigned char smem[];
    pdl_trigger(); pdl_wait();
    unsigned char* sQ = smem;
    unsigned char* stages = smem + FA_BM * FaSmem<D>::STRIDE;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int tpt = FA_BM / a.Gc;                              // tokens per CTA
    // which (entry, first token) is this CTA's?  entries are few: a linear walk.  The last tiles of a prompt see the most
    // keys: they start first, so that the short ones fill the device's tail
    int tile = gridDim.x - 1 - blockIdx.x, e = a.first_entry, q_len = 0;
    for (; e < a.first_entry + a.n_entries; ++e) {
        q_len = a.cu_q[e + 1] - a.cu_q[e];
        const int nt = (q_len + tpt - 1) / tpt;
        if (tile < nt) break;
        tile -= nt;
    }
    if (e >= a.first_entry + a.n_entries) return;
    const int q0 = tile * tpt;
    const int n_tok = min(tpt, q_len - q0);
    const int kh = blockIdx.y / a.chunks, chunk = blockIdx.y % a.chunks;
    const int head0 = kh * (a.QH / a.KH) + chunk * a.Gc;
    const int kv_end = a.kv_len[e];
    const int start_pos = kv_end - q_len;
    const int* bt = a.block_table + (size_t)e * a.max_pages;

    fa_load_q<D>(sQ, a, a.cu_q[e] + q0, n_tok, head0, FA_BM);
    const int pos_min = start_pos + q0, pos_max = start_pos + q0 + n_tok - 1;
    int lo_min = a.window > 0 ? max(0, pos_min - a.window + 1) : 0;
    if (a.chunk > 0) lo_min = max(lo_min, pos_min / a.chunk * a.chunk);
    const int t_begin = lo_min / BN, t_end = pos_max / BN + 1;

    // this thread's two rows
    const int r0 = warp * 16 + (lane >> 2), r1 = r0 + 8;
    const int ti0 = r0 / a.Gc, ti1 = r1 / a.Gc;
    const int pos0 = ti0 < n_tok ? start_pos + q0 + ti0 : -1, pos1 = ti1 < n_tok ? start_pos + q0 + ti1 : -1;
    int lo0 = a.window > 0 ? max(0, pos0 - a.window + 1) : 0, lo1 = a.window > 0 ? max(0, pos1 - a.window + 1) : 0;
    if (a.chunk > 0) { lo0 = max(lo0, max(pos0, 0) / a.chunk * a.chunk); lo1 = max(lo1, max(pos1, 0) / a.chunk * a.chunk); }
    const bool pen = a.r1 != nullptr;
    const int hd0 = head0 + r0 % a.Gc, hd1 = head0 + r1 % a.Gc;
    const float pa0 = pen ? a.r1[hd0] : 0.0f, pb0 = pen ? a.r2[hd0] : 0.0f, pa1 = pen ? a.r1[hd1] : 0.0f, pb1 = pen ? a.r2[hd1] : 0.0f;
    const float* bias0 = a.bias ? a.bias + (size_t)hd0 * a.bias_rows : nullptr;
    const float* bias1 = a.bias ? a.bias + (size_t)hd1 * a.bias_rows : nullptr;
    // keys beyond the last row of this WARP are masked for all its rows: the warp may stop early
    const int warp_last_tok = min(n_tok - 1, (warp * 16 + 15) / a.Gc);
    const int warp_t_end = (warp * 16) / a.Gc < n_tok ? (start_pos + q0 + warp_last_tok) / BN + 1 : 0;

    float o[DO / 8][4];
#pragma unroll
    for (int j = 0; j < DO / 8; ++j) { o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.0f; }
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.0f, 0.0f};

    fa_load_tile<D, VK, BN>(stages, a, bt, kh, t_begin * BN, kv_end);
    cp_async_commit();
    for (int t = t_begin; t < t_end; ++t) {
        const int buf = (t - t_begin) % NST;
        cp_async_wait<0>();
        __syncthreads();                                       // tile t has landed; tile t-1 is no longer read
        if (t + 1 < t_end) fa_load_tile<D, VK, BN>(stages + ((buf + 1) % NST) * STAGE, a, bt, kh, (t + 1) * BN, kv_end);
        cp_async_commit();
        if (t < warp_t_end) {
            const unsigned char* sK = stages + buf * STAGE;
            fa_tile<D, BN / 8, DO>(sQ + warp * 16 * FaSmem<D>::STRIDE, sK, VK ? sK : sK + FaSmem<D, BN>::TILE, 0, t * BN,
                                  pos0, pos1, lo0, lo1, a.scale_log2, o, m, l, pen, pa0, pb0, pa1, pb1,
                                  bias0, bias1, 1, a.bias_rows - 1, a.cap_log2, a.scale_over_cap, a.dv);
        }
    }
    cp_async_wait<0>();
    // join the four threads of a row, normalise, store
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        l[i] += __shfl_xor_sync(0xffffffffu, l[i], 1);
        l[i] += __shfl_xor_sync(0xffffffffu, l[i], 2);
    }
    float f0 = 1.0f, f1 = 1.0f;                                // what the sink's entry into the denominator does to the sums
    if (a.sink) {
        constexpr float LOG2E = 1.4426950408889634f;
        const float s0 = a.sink[hd0] * LOG2E, s1 = a.sink[hd1] * LOG2E;
        const float mf0 = fmaxf(m[0], s0), mf1 = fmaxf(m[1], s1);
        f0 = exp2f(m[0] - mf0); f1 = exp2f(m[1] - mf1);
        l[0] = l[0] * f0 + exp2f(s0 - mf0); l[1] = l[1] * f1 + exp2f(s1 - mf1);
    }
    const float inv0 = l[0] > 0.0f ? a.out_scale / l[0] * f0 : 0.0f, inv1 = l[1] > 0.0f ? a.out_scale / l[1] * f1 : 0.0f;
    const int tok_base = a.cu_q[e] + q0;
    const float* g0 = (a.gate && ti0 < n_tok) ? a.gate + (size_t)(tok_base + ti0) * a.gate_stride + (size_t)hd0 * a.dv : nullptr;
    const float* g1 = (a.gate && ti1 < n_tok) ? a.gate + (size_t)(tok_base + ti1) * a.gate_stride + (size_t)hd1 * a.dv : nullptr;
#pragma unroll
    for (int j = 0; j < DO / 8; ++j) {
        const int dim = j * 8 + 2 * (lane & 3);
        if (dim >= a.dv) continue;
        if (ti0 < n_tok) {
            float x0 = o[j][0] * inv0, x1 = o[j][1] * inv0;
            if (g0) { x0 *= fa_sigmoid(g0[dim]); x1 *= fa_sigmoid(g0[dim + 1]); }
            *reinterpret_cast<uint32_t*>(a.out + ((size_t)(tok_base + ti0) * a.QH + hd0) * a.dv + dim) = pack_bf16(x0, x1);
        }
        if (ti1 < n_tok) {
            float x2 = o[j][2] * inv1, x3 = o[j][3] * inv1;
            if (g1) { x2 *= fa_sigmoid(g1[dim]); x3 *= fa_sigmoid(g1[dim + 1]); }
            *reinterpret_cast<uint32_t*>(a.out + ((size_t)(tok_base + ti1) * a.QH + hd1) * a.dv + dim) = pack_bf16(x2, x3);
        }
    }
}

// ------------------------------------------------------------------------- decode
template <int D, int NST, bool VK>
__global__ void __launch_bounds__(FA_THREADS)
fa_decode_kernel(const FaArgs a) {
    constexpr int STAGE = fa_stage<D, VK>();
    extern __shared__ __align__(16) unsigned char smem[];
    pdl_trigger(); pdl_wait();
    unsigned char* sQ = smem;                                  // 16 rows
    unsigned char* stages = smem + 16 * FaSmem<D>::STRIDE;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int e = a.first_entry + blockIdx.x;                  // a decode entry brings one token: token index = cu_q[e]
    const int kh = blockIdx.y / a.chunks, chunk = blockIdx.y % a.chunks;
    const int head0 = kh * (a.QH / a.KH) + chunk * a.Gc;
    const int split = blockIdx.z;
    const int kv_end = a.kv_len[e];
    const int pos = kv_end - 1;
    int lo = a.window > 0 ? max(0, pos - a.window + 1) : 0;
    if (a.chunk > 0) lo = max(lo, max(pos, 0) / a.chunk * a.chunk);
    const int tok = a.cu_q[e];
    const int* bt = a.block_table + (size_t)e * a.max_pages;
    const int t_lo = lo / FA_BN, t_hi = pos / FA_BN + 1;
    const int per = (t_hi - t_lo + a.n_splits - 1) / a.n_splits;
    const int t_begin = t_lo + split * per, t_end = min(t_hi, t_begin + per);

    fa_load_q<D>(sQ, a, tok, 1, head0, 16);
    const int row0 = lane >> 2;                                // rows >= Gc are padding
    const int pos0 = row0 < a.Gc ? pos : -1, pos1 = row0 + 8 < a.Gc ? pos : -1;
    const bool pen = a.r1 != nullptr;
    const float pa0 = (pen && row0 < a.Gc) ? a.r1[head0 + row0] : 0.0f, pb0 = (pen && row0 < a.Gc) ? a.r2[head0 + row0] : 0.0f;
    const float pa1 = (pen && row0 + 8 < a.Gc) ? a.r1[head0 + row0 + 8] : 0.0f, pb1 = (pen && row0 + 8 < a.Gc) ? a.r2[head0 + row0 + 8] : 0.0f;
    const float* bias0 = (a.bias && row0 < a.Gc) ? a.bias + (size_t)(head0 + row0) * a.bias_rows : nullptr;
    const float* bias1 = (a.bias && row0 + 8 < a.Gc) ? a.bias + (size_t)(head0 + row0 + 8) * a.bias_rows : nullptr;
    float o[D / 8][4];
#pragma unroll
    for (int j = 0; j < D / 8; ++j) { o[j][0] = o[j][1] = o[j][2] = o[j][3] = 0.0f; }
    float m[2] = {-INFINITY, -INFINITY}, l[2] = {0.0f, 0.0f};

#pragma unroll
    for (int i = 0; i < NST - 1; ++i) {
        if (t_begin + i < t_end) fa_load_tile<D, VK>(stages + i * STAGE, a, bt, kh, (t_begin + i) * FA_BN, kv_end);
        cp_async_commit();
    }
    for (int t = t_begin; t < t_end; ++t) {
        const int it = t - t_begin;
        cp_async_wait<NST - 2>();
        __syncthreads();
        if (t + NST - 1 < t_end)
            fa_load_tile<D, VK>(stages + ((it + NST - 1) % NST) * STAGE, a, bt, kh, (t + NST - 1) * FA_BN, kv_end);
        cp_async_commit();
        const unsigned char* sK = stages + (it % NST) * STAGE;
        fa_tile<D, 2>(sQ, sK, VK ? sK : sK + FaSmem<D>::TILE, warp * 16, t * FA_BN, pos0, pos1, lo, lo, a.scale_log2, o, m, l, pen, pa0, pb0, pa1, pb1,
                      bias0, bias1, 1, a.bias_rows - 1, a.cap_log2, a.scale_over_cap, a.dv);
    }
    cp_async_wait<0>();
    __syncthreads();                                           // the stages are free: reuse them for the merge
#pragma unroll
    for (int i = 0; i < 2; ++i) {
        l[i] += __shfl_xor_sync(0xffffffffu, l[i], 1);
        l[i] += __shfl_xor_sync(0xffffffffu, l[i], 2);
    }
    float* sO = reinterpret_cast<float*>(stages);              // [warp][16][D]
    float* sM = sO + FA_WARPS * 16 * D;                        // [warp][16]
    float* sL = sM + FA_WARPS * 16;
#pragma unroll
    for (int j = 0; j < D / 8; ++j) {
        const int dim = j * 8 + 2 * (lane & 3);
        sO[(warp * 16 + row0) * D + dim] = o[j][0]; sO[(warp * 16 + row0) * D + dim + 1] = o[j][1];
        sO[(warp * 16 + row0 + 8) * D + dim] = o[j][2]; sO[(warp * 16 + row0 + 8) * D + dim + 1] = o[j][3];
    }
    if ((lane & 3) == 0) {
        sM[warp * 16 + row0] = m[0]; sM[warp * 16 + row0 + 8] = m[1];
        sL[warp * 16 + row0] = l[0]; sL[warp * 16 + row0 + 8] = l[1];
    }
    __syncthreads();
    // a row's maximum, its warps' factors and its sum once per row (one thread each); then every thread adds columns
    float* sF = sL + FA_WARPS * 16;                            // [warp][16] factor of each warp's part, then [16] 1 / sum
    float* sInv = sF + FA_WARPS * 16;
    const bool sunk = a.sink != nullptr && a.n_splits == 1;    // keys split over CTAs: the merge adds the sink, once
    if (threadIdx.x < a.Gc) {
        const int row = threadIdx.x, head = head0 + row;
        float M = -INFINITY;
#pragma unroll
        for (int w = 0; w < FA_WARPS; ++w) M = fmaxf(M, sM[w * 16 + row]);
        const float sk = sunk ? a.sink[head] * 1.4426950408889634f : -INFINITY;
        if (sunk) M = fmaxf(M, sk);
        float L = 0.0f;
#pragma unroll
        for (int w = 0; w < FA_WARPS; ++w) {
            const float f = M > -INFINITY ? exp2f(sM[w * 16 + row] - M) : 0.0f;   // a warp that saw no key: exp2(-inf) = 0
            sF[w * 16 + row] = f;
            L += sL[w * 16 + row] * f;
        }
        if (sunk && M > -INFINITY) L += exp2f(sk - M);
        sInv[row] = L > 0.0f ? a.out_scale / L : 0.0f;
        if (a.n_splits > 1) {
            const size_t pi = ((size_t)(tok - a.cu_q[a.first_entry]) * a.QH + head) * a.n_splits + split;
            a.part_lse[pi] = L > 0.0f ? M + log2f(L) : -INFINITY;
        }
    }
    __syncthreads();
    for (int row = warp; row < a.Gc; row += FA_WARPS) {
        const int head = head0 + row;
        const float f0 = sF[row], f1 = sF[16 + row], f2 = sF[32 + row], f3 = sF[48 + row], inv = sInv[row];
        static_assert(FA_WARPS == 4, "four parts a row");
        const float* gate = (a.gate && a.n_splits == 1) ? a.gate + (size_t)tok * a.gate_stride + (size_t)head * a.dv : nullptr;
        const size_t pi = ((size_t)(tok - a.cu_q[a.first_entry]) * a.QH + head) * a.n_splits + split;
        for (int dim = lane; dim < a.dv; dim += 32) {
            float O = sO[row * D + dim] * f0;
            O = fmaf(sO[(16 + row) * D + dim], f1, O);
            O = fmaf(sO[(32 + row) * D + dim], f2, O);
            O = fmaf(sO[(48 + row) * D + dim], f3, O);
            float val = O * inv;
            if (a.n_splits == 1) {
                if (gate) val *= fa_sigmoid(gate[dim]);
                a.out[((size_t)tok * a.QH + head) * a.dv + dim] = __float2bfloat16_rn(val);
            } else {
                a.part_o[pi * a.dv + dim] = val;
            }
        }
    }
}

// out[t, h, :] = sum_s w_s o_s / sum_s w_s,  w_s = 2^(lse_s - max lse), splits in ascending order
// sink [QH] (null: none): one more weight 2^(sink log2 e - max) without a value; gate as in FaArgs.
__global__ void fa_merge_kernel(const float* __restrict__ part_o, const float* __restrict__ part_lse, bf16* __restrict__ out,
                                int first_tok, int QH, int d, int n_splits, const float* __restrict__ sink,
                                const float* __restrict__ gate, long long gate_stride) {
    pdl_trigger(); pdl_wait();
    const int t = blockIdx.x, h = blockIdx.y;
    const size_t base = ((size_t)t * QH + h) * n_splits;
    float M = -INFINITY;
    for (int s = 0; s < n_splits; ++s) M = fmaxf(M, part_lse[base + s]);
    const float sk = sink ? sink[h] * 1.4426950408889634f : -INFINITY;
    M = fmaxf(M, sk);
    for (int dim = threadIdx.x; dim < d; dim += blockDim.x) {
        float W = 0.0f, O = 0.0f;
        if (M > -INFINITY) {
            for (int s = 0; s < n_splits; ++s) {
                const float w = exp2f(part_lse[base + s] - M);
                W += w;
                O += w * part_o[(base + s) * d + dim];
            }
            if (sink) W += exp2f(sk - M);
        }
        float val = W > 0.0f ? O / W : 0.0f;
        if (gate) val *= fa_sigmoid(gate[(size_t)(first_tok + t) * gate_stride + (size_t)h * d + dim]);
        out[((size_t)(first_tok + t) * QH + h) * d + dim] = __float2bfloat16_rn(val);
    }
}

// --------------------------------------------------------------------- host side
static int fa_shift(int n) {
    for (int s = 0; s < 31; ++s) if ((1 << s) == n) return s;
    return -1;
}
static int fa_group_chunk(int G) {                             // largest divisor of G that is <= 16
    for (int c = 16; c >= 1; --c) if (G % c == 0) return c;
    return 1;
}

template <int D, bool VK, int BN = FA_BN, int DO = D, int MINB = 1>
static int fa_launch_prefill_as(const FaArgs& a, int n_tiles, cudaStream_t s) {
    const size_t smem = (size_t)FA_BM * FaSmem<D>::STRIDE + 2 * fa_stage<D, VK, BN>();
    static bool done = false;
    if (!done) {
        cudaError_t e = cudaFuncSetAttribute(fa_prefill_kernel<D, VK, BN, DO, MINB>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        done = true;
    }
    return rb_launch(fa_prefill_kernel<D, VK, BN, DO, MINB>, dim3(n_tiles, a.KH * a.chunks), dim3(FA_THREADS), smem, s, a);
}
template <int D>
static int fa_launch_prefill(const FaArgs& a, int n_tiles, cudaStream_t s) {
    if constexpr (D == 256) {
        // Tiles of 32 keys and 192 columns of sums put three CTAs on a SM (168 registers, 66 KB) where the plain shape puts
        // two: more warps to hide the products' latency behind, twice the barriers a key.  It pays once the grid fills the
        // device several times over (measured: 18 % faster at 7 CTAs a SM, 4 % slower at 3.5).
        static int sms = 0;
        if (sms == 0) {
            int dev = 0;
            cudaGetDevice(&dev);
            if (cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || sms <= 0) sms = 148;
        }
        if (a.v_in_k && a.dv <= 192 && (long long)n_tiles * a.KH * a.chunks >= 6LL * sms)
            return fa_launch_prefill_as<256, true, 32, 192, 3>(a, n_tiles, s);
    }
    return a.v_in_k ? fa_launch_prefill_as<D, true>(a, n_tiles, s) : fa_launch_prefill_as<D, false>(a, n_tiles, s);
}
template <int D, int NST, bool VK>
static int fa_launch_decode_as(const FaArgs& a, cudaStream_t s) {
    const size_t pipe = (size_t)NST * fa_stage<D, VK>();
    const size_t merge = ((size_t)FA_WARPS * 16 * (D + 3) + 16) * sizeof(float);    // parts, maxima, sums, factors, 1 / sum
    const size_t smem = 16 * FaSmem<D>::STRIDE + (pipe > merge ? pipe : merge);
    static bool done = false;
    if (!done) {
        cudaError_t e = cudaFuncSetAttribute(fa_decode_kernel<D, NST, VK>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
        done = true;
    }
    return rb_launch(fa_decode_kernel<D, NST, VK>, dim3(a.n_entries, a.KH * a.chunks, a.n_splits), dim3(FA_THREADS), smem, s, a);
}
// (a key tile alone leaves room for one more stage)
template <int D, int NST>
static int fa_launch_decode(const FaArgs& a, cudaStream_t s) {
    return a.v_in_k ? fa_launch_decode_as<D, NST + 1, true>(a, s) : fa_launch_decode_as<D, NST, false>(a, s);
}

// What the soft cap, the sink, values inside the keys and the gate add to the arguments.
struct FaMore {
    float softcap; const float* sink; int v_in_k; const float* gate; long long gate_stride;
};
static int fa_more(FaArgs& a, const FaMore* x, float scale, int d) {
    if (!x) return 0;
    if (x->softcap < 0.0f) RB_REFUSE("attention: a soft cap of %g", (double)x->softcap);
    if (x->v_in_k && a.dv > d) RB_REFUSE("attention: values inside the keys cannot be wider (%d) than the keys (%d)", a.dv, d);
    if (x->softcap > 0.0f) { a.cap_log2 = x->softcap * 1.4426950408889634f; a.scale_over_cap = scale / x->softcap; }
    a.sink = x->sink; a.v_in_k = x->v_in_k; a.gate = x->gate; a.gate_stride = x->gate_stride;
    return 0;
}

static int fa_check(int QH, int KH, int d, int page_size, int max_pages, int dv = 0, const float* bias = nullptr, int bias_rows = 0) {
    if (QH <= 0 || KH <= 0 || QH % KH) RB_REFUSE("attention: %d query heads over %d kv heads", QH, KH);
    if (d <= 0 || d % 8 || d > 256) RB_REFUSE("attention (tensor cores): head_dim %d is not a multiple of 8 up to 256", d);
    if (dv < 0 || dv % 8 || dv > 256) RB_REFUSE("attention (tensor cores): value head size %d is not a multiple of 8 up to 256", dv);
    if (bias && bias_rows <= 0) RB_REFUSE("attention: a distance bias of %d rows", bias_rows);
    if (page_size <= 0 || max_pages <= 0) RB_REFUSE("attention: page_size %d max_pages %d", page_size, max_pages);
    return 0;
}

// Entries [first_entry, first_entry + n_entries) bring q_len >= 1 tokens each; n_tiles = sum over them of
// ceil(q_len / (64 / Gc)) with Gc = rb_fa_group_chunk(QH / KH).
extern "C" int rb_fa_group_chunk(int G) { return fa_group_chunk(G); }

extern "C" int rb_fa_prefill(const void* q, const void* cache, const int* block_table, const int* cu_q, const int* kv_len,
                             void* out, int first_entry, int n_entries, int n_tiles, int QH, int KH, int d, int page_size,
                             int max_pages, int window, float scale, int chunk, const float* r1, const float* r2, float out_scale,
                             int dv, const float* bias, int bias_rows, const FaMore* more, void* stream) {
    if (n_entries <= 0 || n_tiles <= 0) return 0;
    if (fa_check(QH, KH, d, page_size, max_pages, dv, bias, bias_rows)) return -1;
    if (chunk < 0 || (r1 == nullptr) != (r2 == nullptr)) RB_REFUSE("attention: chunk %d, or half a distance penalty", chunk);
    FaArgs a{};
    a.chunk = chunk; a.r1 = r1; a.r2 = r2; a.out_scale = out_scale;
    a.dv = dv > 0 ? dv : d; a.bias = bias; a.bias_rows = bias_rows;
    a.q = (const bf16*)q; a.cache = (const bf16*)cache; a.block_table = block_table; a.cu_q = cu_q; a.kv_len = kv_len;
    a.out = (bf16*)out; a.QH = QH; a.KH = KH; a.d = d; a.page_size = page_size; a.page_shift = fa_shift(page_size); a.max_pages = max_pages; a.window = window;
    a.Gc = fa_group_chunk(QH / KH); a.chunks = (QH / KH) / a.Gc; a.first_entry = first_entry; a.n_entries = n_entries;
    a.n_splits = 1; a.scale_log2 = scale * 1.4426950408889634f;
    if (fa_more(a, more, scale, d)) return -1;
    cudaStream_t s = (cudaStream_t)stream;
    const int wide = a.dv > d ? a.dv : d;                     // the tiles' width serves both sizes
    if (wide <= 32) return fa_launch_prefill<32>(a, n_tiles, s);
    if (wide <= 64) return fa_launch_prefill<64>(a, n_tiles, s);
    if (wide <= 128) return fa_launch_prefill<128>(a, n_tiles, s);
    return fa_launch_prefill<256>(a, n_tiles, s);
}

// Decode entries [first_entry, first_entry + n_entries): one token each.  With n_splits > 1 the scratch
// part_o [n_entries*QH*n_splits*dv] and part_lse [n_entries*QH*n_splits] (floats) must be given.
extern "C" int rb_fa_decode(const void* q, const void* cache, const int* block_table, const int* cu_q, const int* kv_len,
                            void* out, float* part_o, float* part_lse, int first_entry, int n_entries, int first_tok,
                            int n_splits, int QH, int KH, int d, int page_size, int max_pages, int window, float scale,
                            int chunk, const float* r1, const float* r2, float out_scale, int dv, const float* bias,
                            int bias_rows, const FaMore* more, void* stream) {
    if (n_entries <= 0) return 0;
    if (fa_check(QH, KH, d, page_size, max_pages, dv, bias, bias_rows)) return -1;
    if (chunk < 0 || (r1 == nullptr) != (r2 == nullptr)) RB_REFUSE("attention: chunk %d, or half a distance penalty", chunk);
    if (n_splits < 1 || n_splits > 65535) RB_REFUSE("attention: %d splits", n_splits);
    if (n_splits > 1 && (!part_o || !part_lse)) RB_REFUSE("attention: split decoding needs its scratch");
    FaArgs a{};
    a.q = (const bf16*)q; a.cache = (const bf16*)cache; a.block_table = block_table; a.cu_q = cu_q; a.kv_len = kv_len;
    a.out = (bf16*)out; a.part_o = part_o; a.part_lse = part_lse;
    a.chunk = chunk; a.r1 = r1; a.r2 = r2; a.out_scale = out_scale;
    a.dv = dv > 0 ? dv : d; a.bias = bias; a.bias_rows = bias_rows;
    a.QH = QH; a.KH = KH; a.d = d; a.page_size = page_size; a.page_shift = fa_shift(page_size); a.max_pages = max_pages; a.window = window;
    a.Gc = fa_group_chunk(QH / KH); a.chunks = (QH / KH) / a.Gc; a.first_entry = first_entry; a.n_entries = n_entries;
    a.n_splits = n_splits; a.scale_log2 = scale * 1.4426950408889634f;
    if (fa_more(a, more, scale, d)) return -1;
    cudaStream_t s = (cudaStream_t)stream;
    int rc;
    const int wide = a.dv > d ? a.dv : d;
    if (wide <= 32) rc = fa_launch_decode<32, 3>(a, s);
    else if (wide <= 64) rc = fa_launch_decode<64, 3>(a, s);
    else if (wide <= 128) rc = fa_launch_decode<128, 3>(a, s);
    else rc = fa_launch_decode<256, 2>(a, s);
    if (rc || n_splits == 1) return rc;
    return rb_launch(fa_merge_kernel, dim3(n_entries, QH), dim3(128), 0, s, (const float*)part_o, (const float*)part_lse,
                     (bf16*)out, first_tok, QH, a.dv, n_splits, a.sink, a.gate, a.gate_stride);
}
