// One launch for the products of all experts of a mixture, on the warp-level tensor cores (mma.sync m16n8k16,
// bfloat16 operands, float32 accumulation): the bfloat16 engine's form of the grouped product in moe_simt.cu, with
// the same work list (moe_route: the step's (token, k) pairs sorted by expert and cut into row tiles of 64 or 128).
//
// A CTA takes one row tile of one expert and a tile of rows of the expert's matrix (64 x 64 with 4 warps, or 128 x 128
// with 8); it gathers its input rows through the sorted list (pair p reads row p / a_div of A), streams A and W in steps
// of 32 of k through two shared-memory buffers with cp.async, and writes every pair's result to the pair's own row of the
// output.  Epilogues: plain store (float32 or bfloat16), or SiLU(gate) * up for a matrix whose rows
// alternate gate, up: the two lie in neighbouring accumulator columns of one thread, and the output has half the columns.
// Every output element accumulates k in ascending order, whatever else is in the batch.
#include "mma_helpers.cuh"

namespace {
constexpr int BK = 32, PITCH = BK + 8;

struct GroupedMmaParams {
    const void* a; int a_dt; long a_stride; int a_div;             // bfloat16, or float32 rounded to bfloat16 on the way in
    long a_expert_cols;                                            // expert e reads columns from e * a_expert_cols (0: all the same)
    const __nv_bfloat16* w; long w_expert_stride; int w_rows;      // [E][w_rows][K]
    const void* bias; int bias_dt;                                 // [E][w_rows] or null
    void* out; int out_dt; long out_stride; long out_expert_cols;  // expert e writes columns from e * out_expert_cols
    const int* order; const int* tiles; const int* n_tiles;        // tiles == null: every expert takes all dense_rows rows
    int dense_rows, tiles_per_expert;
    int K, gated;                                                  // gated: 0 plain; 1 SiLU(gate) * up of alternating rows; 2 plain, then max(., 0)^2
};

// BM x BN: the CTA's tile; WM x WN warps, each owning (BM / WM) x (BN / WN) of it.  64 x 64 with 2 x 2 warps where an
// expert has few rows (a decode step reads every expert's matrix for a handful of rows: the weights are the cost), 128 x
// 128 with 2 x 4 warps for prompt portions, where the traffic from L2 per multiply-add halves with the tile's edge.
template <int BM, int BN, int WM, int WN>
__global__ void __launch_bounds__(WM * WN * 32) grouped_gemm_mma_kernel(const GroupedMmaParams p) {
    constexpr int THREADS = WM * WN * 32, MT = BM / WM / 16, NT = BN / WN / 8;
    int e, row0, rows;
    if (p.tiles != nullptr) {
        if ((int)blockIdx.y >= p.n_tiles[0]) return;
        e = p.tiles[3 * blockIdx.y]; row0 = p.tiles[3 * blockIdx.y + 1]; rows = p.tiles[3 * blockIdx.y + 2];
    } else {
        e = blockIdx.y / p.tiles_per_expert;
        row0 = (blockIdx.y % p.tiles_per_expert) * BM;
        rows = min(BM, p.dense_rows - row0);
    }
    __shared__ __align__(16) __nv_bfloat16 As[2][BM][PITCH];
    __shared__ __align__(16) __nv_bfloat16 Ws[2][BN][PITCH];
    __shared__ int pair_of_row[BM];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int n0 = blockIdx.x * BN;
    if (tid < BM) pair_of_row[tid] = tid < rows ? (p.order != nullptr ? p.order[row0 + tid] : row0 + tid) : -1;
    __syncthreads();
    const __nv_bfloat16* wbase = p.w + (size_t)e * p.w_expert_stride;
    const size_t a_col0 = (size_t)e * p.a_expert_cols;

    auto load = [&](int buf, int k0) {
#pragma unroll
        for (int q = 0; q < BM * 4 / THREADS; ++q) {
            const int i = tid + q * THREADS;               // BM * 4 chunks of 16 bytes
            const int r = i >> 2, ch = i & 3;
            const int k = k0 + ch * 8;
            const int pr = pair_of_row[r];
            if (pr >= 0 && k < p.K) {
                const size_t ai = (size_t)(pr / p.a_div) * p.a_stride + a_col0 + k;
                if (p.a_dt == RS_BF16) {
                    cp_async16(smem_addr(&As[buf][r][ch * 8]), reinterpret_cast<const __nv_bfloat16*>(p.a) + ai);
                } else {
                    const float4 lo = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(p.a) + ai);
                    const float4 hi = *reinterpret_cast<const float4*>(reinterpret_cast<const float*>(p.a) + ai + 4);
                    uint4 u;
                    u.x = pack_bf16(lo.x, lo.y); u.y = pack_bf16(lo.z, lo.w); u.z = pack_bf16(hi.x, hi.y); u.w = pack_bf16(hi.z, hi.w);
                    *reinterpret_cast<uint4*>(&As[buf][r][ch * 8]) = u;
                }
            } else {
                *reinterpret_cast<uint4*>(&As[buf][r][ch * 8]) = make_uint4(0, 0, 0, 0);
            }
        }
#pragma unroll
        for (int q = 0; q < BN * 4 / THREADS; ++q) {
            const int i = tid + q * THREADS;
            const int r = i >> 2, ch = i & 3;
            const int k = k0 + ch * 8;
            const int gn = n0 + r;
            if (gn < p.w_rows && k < p.K) cp_async16(smem_addr(&Ws[buf][r][ch * 8]), wbase + (size_t)gn * p.K + k);
            else *reinterpret_cast<uint4*>(&Ws[buf][r][ch * 8]) = make_uint4(0, 0, 0, 0);
        }
    };

    float acc[MT][NT][4];
#pragma unroll
    for (int i = 0; i < MT; ++i)
#pragma unroll
        for (int j = 0; j < NT; ++j) { acc[i][j][0] = acc[i][j][1] = acc[i][j][2] = acc[i][j][3] = 0.f; }
    const int m_base = (warp / WN) * (BM / WM), n_base = (warp % WN) * (BN / WN);
    const int a_row = (lane & 7) + 8 * ((lane >> 3) & 1), a_col = 8 * (lane >> 4);
    const int b_row = (lane & 7) + 8 * (lane >> 4), b_col = 8 * ((lane >> 3) & 1);
    const int n_steps = (p.K + BK - 1) / BK;
    load(0, 0);
    cp_async_commit();
    for (int s = 0; s < n_steps; ++s) {
        if (s + 1 < n_steps) {
            load((s + 1) & 1, (s + 1) * BK);
            cp_async_commit();
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
        const int buf = s & 1;
#pragma unroll
        for (int kk = 0; kk < BK; kk += 16) {
            uint32_t a[MT][4], b[NT][2];
#pragma unroll
            for (int i = 0; i < MT; ++i)
                ldmatrix_x4(smem_addr(&As[buf][m_base + i * 16 + a_row][kk + a_col]), a[i][0], a[i][1], a[i][2], a[i][3]);
#pragma unroll
            for (int j = 0; j < NT / 2; ++j)
                ldmatrix_x4(smem_addr(&Ws[buf][n_base + j * 16 + b_row][kk + b_col]), b[2 * j][0], b[2 * j][1], b[2 * j + 1][0],
                            b[2 * j + 1][1]);
#pragma unroll
            for (int i = 0; i < MT; ++i)
#pragma unroll
                for (int j = 0; j < NT; ++j) mma16816(acc[i][j], a[i], b[j][0], b[j][1]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < MT; ++i)
#pragma unroll
        for (int half = 0; half < 2; ++half) {
            const int pr = pair_of_row[m_base + i * 16 + (lane >> 2) + 8 * half];
            if (pr < 0) continue;
#pragma unroll
            for (int j = 0; j < NT; ++j) {
                const int gn = n0 + n_base + j * 8 + (lane & 3) * 2;
                float c0 = acc[i][j][2 * half], c1 = acc[i][j][2 * half + 1];
                if (p.bias != nullptr) {
                    if (gn < p.w_rows) c0 += load_any(p.bias, p.bias_dt, (size_t)e * p.w_rows + gn);
                    if (gn + 1 < p.w_rows) c1 += load_any(p.bias, p.bias_dt, (size_t)e * p.w_rows + gn + 1);
                }
                if (p.gated == 2) {
                    c0 = fmaxf(c0, 0.f); c0 *= c0;
                    c1 = fmaxf(c1, 0.f); c1 *= c1;
                }
                if (p.gated == 1) {
                    if (gn + 1 < p.w_rows) {
                        const float v = silu_mul_fast(c0, c1);
                        const size_t o = (size_t)pr * p.out_stride + (size_t)e * p.out_expert_cols + (gn >> 1);
                        if (p.out_dt == RS_F32) reinterpret_cast<float*>(p.out)[o] = v;
                        else reinterpret_cast<__nv_bfloat16*>(p.out)[o] = __float2bfloat16_rn(v);
                    }
                } else {
                    const size_t o = (size_t)pr * p.out_stride + (size_t)e * p.out_expert_cols + gn;
                    if (p.out_dt == RS_F32) {
                        float* dst = reinterpret_cast<float*>(p.out) + o;
                        if (gn < p.w_rows) dst[0] = c0;
                        if (gn + 1 < p.w_rows) dst[1] = c1;
                    } else {
                        __nv_bfloat16* dst = reinterpret_cast<__nv_bfloat16*>(p.out) + o;
                        if (gn < p.w_rows) dst[0] = __float2bfloat16_rn(c0);
                        if (gn + 1 < p.w_rows) dst[1] = __float2bfloat16_rn(c1);
                    }
                }
            }
        }
}
}  // namespace

// Rows of one expert per CTA: the tile for few rows per expert (large == 0) and the one for prompt portions.
RS_EXPORT int rs_grouped_gemm_mma_rows_per_tile(int large) { return large ? 128 : 64; }

// a: bfloat16 [*, K] rows 16-byte aligned; w: bfloat16 [E][w_rows][K]; out: [pairs, w_rows] (or w_rows / 2 when gated,
// the rows of w alternating gate, up).  K a multiple of 8.
RS_EXPORT int rs_grouped_gemm_mma(const void* a, long a_stride, int a_div, const void* w, long w_expert_stride, int w_rows,
                                  void* out, int out_dt, long out_stride, const int* order, const int* tiles,
                                  const int* n_tiles, int max_tiles, int K, int gated, int large, void* stream) {
    if (max_tiles <= 0 || w_rows <= 0) return 0;
    if (K <= 0 || K % 8 || a_stride % 8 || w_expert_stride % 8 || ((size_t)a & 15) || ((size_t)w & 15) || (gated == 1 && w_rows % 2) || gated < 0 || gated > 2)
        return (int)cudaErrorInvalidValue;
    GroupedMmaParams p{a, RS_BF16, a_stride, a_div, 0, (const __nv_bfloat16*)w, w_expert_stride, w_rows, nullptr, 0, out, out_dt,
                       out_stride, 0, order, tiles, n_tiles, 0, 1, K, gated};
    if (large) grouped_gemm_mma_kernel<128, 128, 2, 4><<<dim3((w_rows + 127) / 128, max_tiles), 256, 0, (cudaStream_t)stream>>>(p);
    else grouped_gemm_mma_kernel<64, 64, 2, 2><<<dim3((w_rows + 63) / 64, max_tiles), 128, 0, (cudaStream_t)stream>>>(p);
    return rs_launch_result();
}

// The block-diagonal product of sequence_parts.cu (rs_block_linear) for more than a few rows, through the same kernel:
// block b is an "expert" that takes every row, reads columns from b * in_bs and writes columns from b * out_bs.
//   out[t, b * out_bs + o] = bias[b, o] + sum_i W[b, o, i] * x[t, b * in_bs + i]
// x: bfloat16, or float32 (rounded to bfloat16 as it enters the product); W: bfloat16 [B, O, I], I a multiple of 8.
RS_EXPORT int rs_block_linear_mma(const void* x, int x_dt, long x_stride, long in_bs, const void* w, const void* bias,
                                  int bias_dt, void* out, int out_dt, long out_stride, long out_bs, int T, int B, int O,
                                  int I, void* stream) {
    if (T <= 0 || B <= 0 || O <= 0) return 0;
    const int align = x_dt == RS_F32 ? 4 : 8;                  // elements per 16 bytes
    if (I <= 0 || I % 8 || x_stride % align || in_bs % align || ((size_t)x & 15) || ((size_t)w & 15))
        return (int)cudaErrorInvalidValue;
    const int bm = T > 256 ? 128 : 64;
    const int tiles_per = (T + bm - 1) / bm;
    GroupedMmaParams p{x, x_dt, x_stride, 1, in_bs, (const __nv_bfloat16*)w, (long)O * I, O, bias, bias_dt, out, out_dt, out_stride,
                       out_bs, nullptr, nullptr, nullptr, T, tiles_per, I, 0};
    if (bm == 128) grouped_gemm_mma_kernel<128, 128, 2, 4><<<dim3((O + 127) / 128, tiles_per * B), 256, 0, (cudaStream_t)stream>>>(p);
    else grouped_gemm_mma_kernel<64, 64, 2, 2><<<dim3((O + 63) / 64, tiles_per * B), 128, 0, (cudaStream_t)stream>>>(p);
    return rs_launch_result();
}
