// One small matrix per head, all heads in one launch:  y[t, h, :] = W[h] x[t, h, :],  W [H, out, in] bfloat16.
//
// The maps that latent attention moves to the query's side (keys' map on the plain part of q, values' map on the
// attention's output) are H products of 64..512 inputs and outputs each: a few FLOPs per byte, so the kernel is
// bound by reading x and writing y once, not by the tensor pipe.  A CTA owns 64 tokens x 64 outputs of one head and
// walks the inputs 64 at a time through two cp.async stages; four warps of 16 rows each run mma.sync m16n8k16 on
// ldmatrix fragments (x rows and W rows are both contiguous over the inputs: the "row.col" form as it lies).  Rows
// beyond T, inputs beyond n_in and outputs beyond n_out are zero-filled on the way in and skipped on the way out.
// A row's sums do not depend on the other rows of its tile or on T: a token's result is the same alone and in a batch.
//
// Optionally the kernel also carries a tail along: `tail` columns that follow a head's inputs in x are copied behind
// the head's outputs in y with their first `rot` dimensions rotated in neighbouring pairs (2i, 2i + 1) by
// position * freq[i], cosine and sine times `mag` - the rotated part of a query head, which passes the map unchanged.
// And optionally a gate: float rows [T, H * n_out] (row stride of their own) whose sigmoid multiplies the outputs.
#include "common.cuh"

#define HG_BM 64
#define HG_BN 64
#define HG_BK 64
#define HG_THREADS 128
#define HG_STRIDE (HG_BK * 2 + 16)              // bytes per tile row: 16 bytes of padding keep ldmatrix conflict-free
#define HG_TILE (HG_BM * HG_STRIDE)

__device__ __forceinline__ void hg_cp16(void* dst, const void* src, int src_bytes) {
    const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(src), "r"(src_bytes) : "memory");
}
__device__ __forceinline__ void hg_ldsm(uint32_t (&r)[4], const void* p) {
    const uint32_t a = (uint32_t)__cvta_generic_to_shared(p);
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];" : "=r"(r[0]), "=r"(r[1]), "=r"(r[2]), "=r"(r[3]) : "r"(a));
}
__device__ __forceinline__ void hg_mma(float (&c)[4], const uint32_t (&a)[4], uint32_t b0, uint32_t b1) {
    asm volatile("mma.sync.aligned.m16n8k16.row.col.f32.bf16.bf16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
                 : "+f"(c[0]), "+f"(c[1]), "+f"(c[2]), "+f"(c[3]) : "r"(a[0]), "r"(a[1]), "r"(a[2]), "r"(a[3]), "r"(b0), "r"(b1));
}

__global__ void __launch_bounds__(HG_THREADS)
heads_linear_mma_kernel(const bf16* __restrict__ x, long long x_row, long long x_head, const bf16* __restrict__ w, bf16* __restrict__ y,
                        long long y_row, long long y_head, int T, int n_in, int n_out, int tail, int rot,
                        const int* __restrict__ positions, const float* __restrict__ freq, float mag,
                        const float* __restrict__ gate, long long gate_row) {
    __shared__ __align__(16) unsigned char smem[2 * 2 * HG_TILE];
    pdl_trigger();
    pdl_wait();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int t0 = blockIdx.x * HG_BM, o0 = blockIdx.y * HG_BN, h = blockIdx.z;
    const bf16* xh = x + (size_t)h * x_head;
    const bf16* wh = w + (size_t)h * n_out * n_in;
    const int n_k = (n_in + HG_BK - 1) / HG_BK;

    // a thread copies the same 16-byte column of rows r, r + 16, ... of both tiles
    const int c16 = threadIdx.x & 7, r_first = threadIdx.x >> 3;
    auto load = [&](int stage, int k0) {
        unsigned char* sA = smem + stage * 2 * HG_TILE;
        unsigned char* sB = sA + HG_TILE;
        const int k = k0 + c16 * 8;
        const bool k_in = k < n_in;                                  // n_in is a multiple of 8: a chunk is inside or outside
#pragma unroll
        for (int i = 0; i < HG_BM / 16; ++i) {
            const int r = r_first + i * 16;
            const bool a_in = k_in && t0 + r < T, b_in = k_in && o0 + r < n_out;
            hg_cp16(sA + r * HG_STRIDE + c16 * 16, a_in ? (const void*)(xh + (size_t)(t0 + r) * x_row + k) : (const void*)x, a_in ? 16 : 0);
            hg_cp16(sB + r * HG_STRIDE + c16 * 16, b_in ? (const void*)(wh + (size_t)(o0 + r) * n_in + k) : (const void*)w, b_in ? 16 : 0);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };

    float acc[HG_BN / 8][4];
#pragma unroll
    for (int j = 0; j < HG_BN / 8; ++j) acc[j][0] = acc[j][1] = acc[j][2] = acc[j][3] = 0.0f;
    load(0, 0);
    for (int ki = 0; ki < n_k; ++ki) {
        if (ki + 1 < n_k) {
            load((ki + 1) & 1, (ki + 1) * HG_BK);
            asm volatile("cp.async.wait_group 1;" ::: "memory");
        } else {
            asm volatile("cp.async.wait_group 0;" ::: "memory");
        }
        __syncthreads();
        const unsigned char* sA = smem + (ki & 1) * 2 * HG_TILE + warp * 16 * HG_STRIDE;
        const unsigned char* sB = smem + (ki & 1) * 2 * HG_TILE + HG_TILE;
#pragma unroll
        for (int ks = 0; ks < HG_BK / 16; ++ks) {
            uint32_t a[4];
            hg_ldsm(a, sA + ((lane & 7) + 8 * ((lane >> 3) & 1)) * HG_STRIDE + (ks * 16 + 8 * (lane >> 4)) * 2);
#pragma unroll
            for (int jp = 0; jp < HG_BN / 16; ++jp) {
                uint32_t b[4];
                hg_ldsm(b, sB + (jp * 16 + (lane & 7) + 8 * (lane >> 4)) * HG_STRIDE + (ks * 16 + 8 * ((lane >> 3) & 1)) * 2);
                hg_mma(acc[2 * jp], a, b[0], b[1]);
                hg_mma(acc[2 * jp + 1], a, b[2], b[3]);
            }
        }
        __syncthreads();                                             // the stage may be filled again
    }

    // rows lane / 4 and lane / 4 + 8 of the warp's 16, columns 2 (lane % 4) and the next of every 8
    bf16* yh = y + (size_t)h * y_head;
    const bool pairs_ok = ((y_row | y_head) & 1) == 0 && (((uintptr_t)y) & 3) == 0;
#pragma unroll
    for (int half = 0; half < 2; ++half) {
        const int t = t0 + warp * 16 + (lane >> 2) + half * 8;
        if (t >= T) continue;
        bf16* yr = yh + (size_t)t * y_row;
#pragma unroll
        for (int j = 0; j < HG_BN / 8; ++j) {
            const int o = o0 + j * 8 + 2 * (lane & 3);
            float v0 = acc[j][half * 2], v1 = acc[j][half * 2 + 1];
            if (gate) {                                              // the output gate: times sigmoid(gate[t, h, o])
                const float* gr = gate + (size_t)t * gate_row + (size_t)h * n_out;
                if (o < n_out) v0 *= 1.0f / (1.0f + expf(-gr[o]));
                if (o + 1 < n_out) v1 *= 1.0f / (1.0f + expf(-gr[o + 1]));
            }
            if (o + 1 < n_out && pairs_ok) *reinterpret_cast<__nv_bfloat162*>(yr + o) = __floats2bfloat162_rn(v0, v1);
            else {
                if (o < n_out) yr[o] = __float2bfloat16_rn(v0);
                if (o + 1 < n_out) yr[o + 1] = __float2bfloat16_rn(v1);
            }
        }
    }

    if (tail > 0 && blockIdx.y == 0) {
        const int pairs = (tail + 1) / 2;
        const int rows = min(HG_BM, T - t0);
        for (int i = threadIdx.x; i < rows * pairs; i += HG_THREADS) {
            const int t = t0 + i / pairs, p = i % pairs, d = 2 * p;
            const bf16* s = xh + (size_t)t * x_row + n_in;
            bf16* dst = yh + (size_t)t * y_row + n_out;
            float u = __bfloat162float(s[d]);
            if (d + 1 < tail) {
                float v = __bfloat162float(s[d + 1]);
                if (d + 1 < rot) {
                    float sn, cs;
                    sincosf((float)positions[t] * freq[p], &sn, &cs);
                    cs *= mag; sn *= mag;
                    const float a = u * cs - v * sn, b = v * cs + u * sn;
                    u = a; v = b;
                }
                dst[d + 1] = __float2bfloat16_rn(v);
            }
            dst[d] = __float2bfloat16_rn(u);
        }
    }
}

// x [T, H, n_in (+ tail)] and y [T, H, n_out (+ tail)] bfloat16 with row and head strides of their own (in elements; x's
// multiples of 8 and x 16-byte aligned); w [H, n_out, n_in] contiguous bfloat16, 16-byte aligned; n_in a multiple of 8.
extern "C" int rb_heads_linear_mma(const void* x, long long x_row, long long x_head, const void* w, void* y, long long y_row,
                                   long long y_head, int T, int H, int n_in, int n_out, int tail, int rot, const int* positions,
                                   const float* freq, float mag, const float* gate, long long gate_row, void* stream) {
    if (T <= 0 || H <= 0 || n_out <= 0) return 0;
    if (n_in <= 0 || n_in % 8) RB_REFUSE("heads_linear (mma): %d inputs a head (a multiple of 8)", n_in);
    if ((x_row % 8) || (x_head % 8) || ((uintptr_t)x & 15) || ((uintptr_t)w & 15))
        RB_REFUSE("heads_linear (mma): x and w must be 16-byte aligned, x's strides multiples of 8");
    if (tail < 0 || rot < 0 || rot % 2 || rot > tail || (rot > 0 && (!positions || !freq)))
        RB_REFUSE("heads_linear (mma): a tail of %d with %d rotated dimensions", tail, rot);
    if (H > 65535 || rb_ceil_div(n_out, HG_BN) > 65535) RB_REFUSE("heads_linear (mma): %d heads, %d outputs", H, n_out);
    return rb_launch(heads_linear_mma_kernel, dim3(rb_ceil_div(T, HG_BM), rb_ceil_div(n_out, HG_BN), H), dim3(HG_THREADS), 0,
                     (cudaStream_t)stream, (const bf16*)x, x_row, x_head, (const bf16*)w, (bf16*)y, y_row, y_head, T, n_in, n_out,
                     tail, rot, positions, freq, mag, gate, gate_row);
}
