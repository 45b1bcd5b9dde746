// The plain attention over the paged cache: any number of new tokens per request,
// causal, grouped heads, optional window.  One warp per (token, query head) walks the
// keys of its request in ascending order, in blocks of 32 that are aligned to absolute
// positions, with one online-softmax update per block.  The sequence of operations for
// a token depends only on its position (and the window), never on how the request was
// cut into steps, on the batch, or on the page size - so this kernel gives the same
// bits under every cut.  It is the attention of the 32-bit path and the yardstick of
// the faster bfloat16 kernels.
// Beyond the plain form it takes: a value head size of its own (dv != d), a chunk mask (a token sees the
// keys of its own chunk of `chunk` positions, counted from position 0), a logarithmic distance penalty per
// query head (score -= r1[h] * ln(1 + r2[h] * (i - j))), a learned bias by distance (score += bias[h][min(i - j,
// rows - 1)], a float table [QH, rows] whose last column stands for every greater distance), and a factor on the output.
// Further options: scores squashed to cap * tanh(score / cap) (softcap > 0); a sink per query head, a number that joins
// the softmax's denominator as exp(sink[h]) and brings no value; values that are the first dv columns of the key rows
// (v_in_k: a page then holds keys only, [KH][page_size][d]); and a gate on the output, out *= sigmoid(gate[t][h * dv + i])
// (float rows with a stride of their own).
// (reference semantics: crates/cuda/kernels/decode_gqa_kernels.cu:99-136 page lookup
//  page[t/block_len]; decode_flash_kernels.cu:212-349 max/exp/sum/PV in f32.)
#include "common.cuh"

#define RA_WARPS 4
#define RA_MAX_D 512

// q        [T, QH, d];  out [T, QH, dv]
// cache    one layer: [page][ K: [KH][page_size][d] | V: [KH][page_size][dv] ]   (dv == d: [page][2][KH][page_size][d])
// block_table [rows, max_pages] (page id of the i-th page of a request's row)
// tok_row  [T] row of block_table for token t;  positions [T] absolute position of token t
// A token at position p attends keys max(0, p-window+1) .. p  (window <= 0: all of them); with chunk > 0 also
// only keys from floor(p / chunk) * chunk on.
template <typename TA, typename TC>
__global__ void __launch_bounds__(RA_WARPS * 32)
paged_attention_ref_kernel(const TA* __restrict__ q, const TC* __restrict__ cache,
                           const int* __restrict__ block_table, const int* __restrict__ tok_row,
                           const int* __restrict__ positions, TA* __restrict__ out,
                           int QH, int KH, int d, int dv, int page_size, int max_pages, int window, float scale,
                           int chunk, const float* __restrict__ r1, const float* __restrict__ r2, float out_scale,
                           const float* __restrict__ bias, int bias_rows, float softcap, const float* __restrict__ sink,
                           int v_in_k, const float* __restrict__ gate, long long gate_stride) {
    pdl_trigger(); pdl_wait();
    extern __shared__ float qs_all[];                         // RA_WARPS * d floats
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t = blockIdx.x;
    const int hq = blockIdx.y * RA_WARPS + warp;
    if (hq >= QH) return;                                     // no block-wide barrier below
    float* qs = qs_all + warp * d;
    const TA* qp = q + ((size_t)t * QH + hq) * d;
    for (int i = lane; i < d; i += 32) qs[i] = to_f32(qp[i]);
    __syncwarp();
    const int kh = hq / (QH / KH);
    const int pos = positions[t];
    int lo = (window > 0 && pos - window + 1 > 0) ? pos - window + 1 : 0;
    if (chunk > 0) lo = max(lo, pos / chunk * chunk);
    const float pen1 = r1 ? r1[hq] : 0.0f, pen2 = r1 ? r2[hq] : 0.0f;
    const int* bt = block_table + (size_t)tok_row[t] * max_pages;
    const size_t head_stride = (size_t)page_size * d;         // one (page, k, head) tile
    const size_t vhead_stride = v_in_k ? head_stride : (size_t)page_size * dv;   // one (page, v, head) tile
    const size_t page_stride = v_in_k ? (size_t)KH * head_stride : (size_t)KH * (head_stride + vhead_stride);
    const size_t v_offset = v_in_k ? 0 : (size_t)KH * head_stride;                // values behind the keys, or inside them
    const int v_row = v_in_k ? d : dv;
    const float inv_cap = softcap > 0.0f ? 1.0f / softcap : 0.0f;

    constexpr int NACC = RA_MAX_D / 32;
    float acc[NACC];
#pragma unroll
    for (int i = 0; i < NACC; ++i) acc[i] = 0.0f;
    float m = -INFINITY, l = 0.0f;

    for (int b0 = (lo / 32) * 32; b0 <= pos; b0 += 32) {
        const int key = b0 + lane;
        bool valid = key >= lo && key <= pos;
        float s = -INFINITY;
        const TC* vrow = nullptr;
        const int page = (valid && key / page_size < max_pages) ? bt[key / page_size] : -1;
        valid = valid && page >= 0;                            // a page that is not held: an inert padding row
        if (valid) {
            const int off = key % page_size;
            const TC* krow = cache + (size_t)page * page_stride + (size_t)kh * head_stride + (size_t)off * d;
            vrow = cache + (size_t)page * page_stride + v_offset + (size_t)kh * vhead_stride + (size_t)off * v_row;
            float dot = 0.0f;
            for (int i = 0; i < d; ++i) dot = fmaf(qs[i], to_f32(krow[i]), dot);
            s = dot * scale;
            if (softcap > 0.0f) s = softcap * tanhf(s * inv_cap);
            if (r1) s -= pen1 * log1pf(pen2 * (float)(pos - key));
            if (bias) s += bias[(size_t)hq * bias_rows + min(pos - key, bias_rows - 1)];
        }
        const float bm = warp_max(s);
        if (bm == -INFINITY) continue;                         // no key in this block (warp-uniform)
        const float m_new = fmaxf(m, bm);
        const float corr = expf(m - m_new);                    // first block: exp(-inf) = 0
        const float p = valid ? expf(s - m_new) : 0.0f;
        l = l * corr + warp_sum(p);
#pragma unroll
        for (int i = 0; i < NACC; ++i) acc[i] *= corr;
        for (int j = 0; j < 32; ++j) {
            const float pj = __shfl_sync(0xffffffffu, p, j);
            const unsigned long long vj = __shfl_sync(0xffffffffu, (unsigned long long)vrow, j);
            if (vj == 0ull) continue;                          // warp-uniform
            const TC* vr = (const TC*)vj;
#pragma unroll
            for (int i = 0; i < NACC; ++i) {
                const int dim = lane + 32 * i;
                if (dim < dv) acc[i] = fmaf(pj, to_f32(vr[dim]), acc[i]);
            }
        }
        m = m_new;
    }
    if (sink) {                                                // one more term in the denominator, no value
        const float sk = sink[hq];
        const float m_new = fmaxf(m, sk);
        const float corr = expf(m - m_new);
        l = l * corr + expf(sk - m_new);
#pragma unroll
        for (int i = 0; i < NACC; ++i) acc[i] *= corr;
    }
    const float inv = l > 0.0f ? 1.0f / l : 0.0f;
    TA* op = out + ((size_t)t * QH + hq) * dv;
    const float* gp = gate ? gate + (size_t)t * gate_stride + (size_t)hq * dv : nullptr;
#pragma unroll
    for (int i = 0; i < NACC; ++i) {
        const int dim = lane + 32 * i;
        if (dim < dv) {
            float val = out_scale == 1.0f ? acc[i] * inv : acc[i] * inv * out_scale;
            if (gp) val *= 1.0f / (1.0f + expf(-gp[dim]));
            op[dim] = from_f32<TA>(val);
        }
    }
}

// dv: the value heads' size (0: as d).  chunk 0: no chunk mask.  r1, r2 [QH] float: the distance penalty (null: none).
// bias [QH, bias_rows] float: the bias by distance (null: none).  softcap 0: none.  sink [QH] float (null: none).
// v_in_k != 0: the values are the first dv columns of the keys.  gate: float rows of stride gate_stride (null: none).
extern "C" int rb_paged_attention_ref(const void* q, const void* cache, int dtype,
                                      const int* block_table, const int* tok_row, const int* positions,
                                      void* out, int n_tokens, int QH, int KH, int d, int page_size,
                                      int max_pages, int window, float scale, int dv, int chunk, const float* r1,
                                      const float* r2, float out_scale, const float* bias, int bias_rows, float softcap,
                                      const float* sink, int v_in_k, const float* gate, long long gate_stride, void* stream) {
    if (n_tokens <= 0) return 0;
    if (dv <= 0) dv = d;
    if (QH <= 0 || KH <= 0 || QH % KH != 0) RB_REFUSE("attention: %d query heads over %d kv heads", QH, KH);
    if (d <= 0 || d > RA_MAX_D || dv > RA_MAX_D) RB_REFUSE("attention: head sizes %d, %d (supported: 1..%d)", d, dv, RA_MAX_D);
    if (page_size <= 0 || max_pages <= 0) RB_REFUSE("attention: page_size %d max_pages %d", page_size, max_pages);
    if (chunk < 0 || (r1 == nullptr) != (r2 == nullptr)) RB_REFUSE("attention: chunk %d, or half a distance penalty", chunk);
    if (bias && bias_rows <= 0) RB_REFUSE("attention: a distance bias of %d rows", bias_rows);
    if (v_in_k && dv > d) RB_REFUSE("attention: values inside the keys cannot be wider (%d) than the keys (%d)", dv, d);
    if (softcap < 0.0f) RB_REFUSE("attention: a soft cap of %g", (double)softcap);
    cudaStream_t s = (cudaStream_t)stream;
    dim3 grid(n_tokens, rb_ceil_div(QH, RA_WARPS));
    const size_t smem = (size_t)RA_WARPS * d * sizeof(float);
    if (dtype == RB_F32)
        return rb_launch(paged_attention_ref_kernel<float, float>, grid, dim3(RA_WARPS * 32), smem, s,
            (const float*)q, (const float*)cache, block_table, tok_row, positions, (float*)out,
            QH, KH, d, dv, page_size, max_pages, window, scale, chunk, r1, r2, out_scale, bias, bias_rows,
            softcap, sink, v_in_k, gate, gate_stride);
    if (dtype == RB_BF16)
        return rb_launch(paged_attention_ref_kernel<bf16, bf16>, grid, dim3(RA_WARPS * 32), smem, s,
            (const bf16*)q, (const bf16*)cache, block_table, tok_row, positions, (bf16*)out,
            QH, KH, d, dv, page_size, max_pages, window, scale, chunk, r1, r2, out_scale, bias, bias_rows,
            softcap, sink, v_in_k, gate, gate_stride);
    RB_REFUSE("attention: dtype %d", dtype);
}
