// Mixture of experts whose choice is known before the layer runs (a table from token id to expert ids), on CUDA
// cores with float32 accumulation, for both engines:
//   * moe_route: the step's (token, k) pairs sorted by expert, entirely on the device: counts, offsets, the list of
//     row tiles (expert, first sorted row, rows) that the grouped products walk;
//   * grouped_linear: one launch for all experts; a CTA takes one row tile of one expert and one tile of output
//     columns, gathers its input rows through the sorted list and writes each pair's result to the pair's own row.
//     Epilogues: plain store, or SiLU(gate) * up with gate rows [0, N) and up rows [N, 2N) of the expert's matrix.
//     A tile of at most 8 rows takes the row-streaming form (a warp per output column, the expert's matrix read
//     once, coalesced); larger tiles the 64 x 64 register-tiled form;
//   * moe_combine: out[t] = sum_k pair_out[t, k] * weight + sigmoid(h[t] . w_gate) * shared[t], the sum over k in
//     ascending k, so a token's result does not depend on the batch.
// Every pair's row is computed with k ascending whatever else is in the batch.
#include "common.cuh"
#include <math.h>

namespace {
__device__ __forceinline__ void store_any(void* p, int dt, size_t i, float v) {
    if (dt == RS_F32) reinterpret_cast<float*>(p)[i] = v;
    else reinterpret_cast<__nv_bfloat16*>(p)[i] = __float2bfloat16_rn(v);
}
constexpr int MAX_EXPERTS = 4096;
}  // namespace

// order[P]: pair ids (t * top + k) grouped by expert; tiles[i] = (expert, first row in order, rows); n_tiles[0].
__global__ void __launch_bounds__(1024) moe_route_kernel(const int* __restrict__ ids, const int* __restrict__ table, int V,
                                                         int top, int E, int n_tokens, int rows_per_tile,
                                                         int* __restrict__ order, int* __restrict__ tiles,
                                                         int* __restrict__ n_tiles, int max_tiles, int* status) {
    __shared__ int counts[MAX_EXPERTS];
    __shared__ int cursor[MAX_EXPERTS];
    const int P = n_tokens * top;
    for (int e = threadIdx.x; e < E; e += blockDim.x) counts[e] = 0;
    __syncthreads();
    for (int pr = threadIdx.x; pr < P; pr += blockDim.x) {
        int id = ids != nullptr ? ids[pr / top] : pr / top;        // without ids the table has one row per token of the step
        if (id < 0 || id >= V) { atomicOr(status, RS_STATUS_BAD_TOKEN); id = 0; }
        int e = table[(size_t)id * top + pr % top];
        if (e < 0 || e >= E) { atomicOr(status, RS_STATUS_BAD_PLAN); e = 0; }
        atomicAdd(&counts[e], 1);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int off = 0, nt = 0;
        for (int e = 0; e < E; ++e) {
            cursor[e] = off;
            for (int r0 = 0; r0 < counts[e]; r0 += rows_per_tile) {
                if (nt < max_tiles) {
                    tiles[3 * nt] = e; tiles[3 * nt + 1] = off + r0; tiles[3 * nt + 2] = min(rows_per_tile, counts[e] - r0);
                }
                ++nt;
            }
            off += counts[e];
        }
        if (nt > max_tiles) { atomicOr(status, RS_STATUS_BAD_PLAN); nt = max_tiles; }
        n_tiles[0] = nt;
    }
    __syncthreads();
    // Where a pair lands within its expert's rows changes no value: every pair's row is computed by itself.
    for (int pr = threadIdx.x; pr < P; pr += blockDim.x) {
        int id = ids != nullptr ? ids[pr / top] : pr / top;
        if (id < 0 || id >= V) id = 0;
        int e = table[(size_t)id * top + pr % top];
        if (e < 0 || e >= E) e = 0;
        order[atomicAdd(&cursor[e], 1)] = pr;
    }
}

RS_EXPORT int rs_moe_route(const int* ids, const int* table, int V, int top, int E, int n_tokens, int rows_per_tile,
                           int* order, int* tiles, int* n_tiles, int max_tiles, int* status, void* stream) {
    if (n_tokens <= 0) return 0;
    if (E <= 0 || E > MAX_EXPERTS || top <= 0 || rows_per_tile <= 0) return (int)cudaErrorInvalidValue;
    moe_route_kernel<<<1, 1024, 0, (cudaStream_t)stream>>>(ids, table, V, top, E, n_tokens, rows_per_tile, order, tiles,
                                                           n_tiles, max_tiles, status);
    return rs_launch_result();
}

namespace {
constexpr int GL_BM = 64, GL_BN = 64, GL_BK = 16;

struct GroupedParams {
    const void* a; int a_dt; long a_stride; int a_div;       // input row of a pair = pair / a_div
    const void* w; int w_dt; long w_expert_stride;           // [E][rows][K], rows = N (plain) or 2N (gated)
    void* out; int out_dt; long out_stride;                  // [P, N]
    const int* order; const int* tiles; const int* n_tiles;
    int N, K, gated;          // gated: 0 plain; 1 gate rows [0, N) and up rows [N, 2N); 2 gate row 2n, up row 2n + 1
    int relu2;                // plain products only: out = max(a W.T, 0)^2
};

__device__ __forceinline__ float relu_squared(float v) { v = fmaxf(v, 0.f); return v * v; }

__device__ __forceinline__ size_t gate_row(const GroupedParams& p, int n) { return p.gated == 2 ? 2 * (size_t)n : (size_t)n; }
__device__ __forceinline__ size_t up_row(const GroupedParams& p, int n) { return p.gated == 2 ? 2 * (size_t)n + 1 : (size_t)p.N + n; }

__device__ __forceinline__ float silu_exact(float g) { return g / (1.0f + expf(-g)); }

// 64 x 64 register-tiled form
__global__ void __launch_bounds__(256) grouped_linear_tile_kernel(const GroupedParams p) {
    if ((int)blockIdx.y >= p.n_tiles[0]) return;
    __shared__ float As[GL_BK][GL_BM + 1];
    __shared__ float Ws[GL_BK][GL_BN + 1];
    __shared__ float Us[GL_BK][GL_BN + 1];
    __shared__ int pair_of_row[GL_BM];
    const int e = p.tiles[3 * blockIdx.y], row0 = p.tiles[3 * blockIdx.y + 1], rows = p.tiles[3 * blockIdx.y + 2];
    const int tid = threadIdx.x, n0 = blockIdx.x * GL_BN;
    const int tx = tid % 16, ty = tid / 16;
    if (tid < GL_BM) pair_of_row[tid] = tid < rows ? p.order[row0 + tid] : -1;
    __syncthreads();
    float acc[4][4], accu[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) { acc[i][j] = 0.f; accu[i][j] = 0.f; }
    const size_t wb = (size_t)e * p.w_expert_stride;
    for (int k0 = 0; k0 < p.K; k0 += GL_BK) {
#pragma unroll
        for (int q = 0; q < 4; ++q) {
            const int idx = tid + q * 256;
            const int r = idx / GL_BK, kk = idx % GL_BK;
            const int gk = k0 + kk, gn = n0 + r;
            const int pr = pair_of_row[r];
            As[kk][r] = (pr >= 0 && gk < p.K) ? load_any(p.a, p.a_dt, (size_t)(pr / p.a_div) * p.a_stride + gk) : 0.f;
            const bool ok = gn < p.N && gk < p.K;
            Ws[kk][r] = ok ? load_any(p.w, p.w_dt, wb + gate_row(p, gn) * p.K + gk) : 0.f;
            if (p.gated) Us[kk][r] = ok ? load_any(p.w, p.w_dt, wb + up_row(p, gn) * p.K + gk) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < GL_BK; ++kk) {
            float a[4], w[4], u[4];
#pragma unroll
            for (int i = 0; i < 4; ++i) a[i] = As[kk][ty * 4 + i];
#pragma unroll
            for (int j = 0; j < 4; ++j) { w[j] = Ws[kk][tx * 4 + j]; u[j] = p.gated ? Us[kk][tx * 4 + j] : 0.f; }
#pragma unroll
            for (int i = 0; i < 4; ++i)
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    acc[i][j] = fmaf(a[i], w[j], acc[i][j]);
                    if (p.gated) accu[i][j] = fmaf(a[i], u[j], accu[i][j]);
                }
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const int pr = pair_of_row[ty * 4 + i];
        if (pr < 0) continue;
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int gn = n0 + tx * 4 + j;
            if (gn >= p.N) continue;
            const float v = p.gated ? silu_exact(acc[i][j]) * accu[i][j] : (p.relu2 ? relu_squared(acc[i][j]) : acc[i][j]);
            store_any(p.out, p.out_dt, (size_t)pr * p.out_stride + gn, v);
        }
    }
}

// row-streaming form for tiles of at most 8 rows: the rows sit in shared memory as float32, a warp owns output
// columns and reads their weight rows once, lanes striding over k.
constexpr int GR_ROWS = 8, GR_COLS = 32, GR_KC = 1024;

__global__ void __launch_bounds__(256) grouped_linear_rows_kernel(const GroupedParams p) {
    if ((int)blockIdx.y >= p.n_tiles[0]) return;
    __shared__ float As[GR_ROWS][GR_KC];
    __shared__ int pair_of_row[GR_ROWS];
    const int e = p.tiles[3 * blockIdx.y], row0 = p.tiles[3 * blockIdx.y + 1], rows = p.tiles[3 * blockIdx.y + 2];
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int n0 = blockIdx.x * GR_COLS;
    if (tid < GR_ROWS) pair_of_row[tid] = tid < rows ? p.order[row0 + tid] : -1;
    constexpr int CPW = GR_COLS / 8;                          // columns per warp
    float acc[CPW][GR_ROWS], accu[CPW][GR_ROWS];
#pragma unroll
    for (int c = 0; c < CPW; ++c)
#pragma unroll
        for (int r = 0; r < GR_ROWS; ++r) { acc[c][r] = 0.f; accu[c][r] = 0.f; }
    const size_t wb = (size_t)e * p.w_expert_stride;
    const bool vec = p.w_dt == RS_BF16 && p.K % 8 == 0 && p.w_expert_stride % 8 == 0 && ((size_t)p.w & 15) == 0;
    for (int k0 = 0; k0 < p.K; k0 += GR_KC) {
        __syncthreads();
        const int kc = min(GR_KC, p.K - k0);
        for (int i = tid; i < GR_ROWS * kc; i += 256) {
            const int r = i / kc, kk = i % kc;
            const int pr = pair_of_row[r];
            As[r][kk] = pr >= 0 ? load_any(p.a, p.a_dt, (size_t)(pr / p.a_div) * p.a_stride + k0 + kk) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int c = 0; c < CPW; ++c) {
            const int gn = n0 + warp * CPW + c;
            if (gn >= p.N) continue;
            const size_t wrow = wb + gate_row(p, gn) * p.K + k0, urow = wb + up_row(p, gn) * p.K + k0;
            if (vec) {
                // eight bfloat16 weights per lane and load (16 bytes), the rows' values from shared memory
                const __nv_bfloat16* wp = reinterpret_cast<const __nv_bfloat16*>(p.w);
                for (int kk = lane * 8; kk < kc; kk += 256) {
                    const uint4 wv = *reinterpret_cast<const uint4*>(wp + wrow + kk);
                    uint4 uv = make_uint4(0, 0, 0, 0);
                    if (p.gated) uv = *reinterpret_cast<const uint4*>(wp + urow + kk);
                    const __nv_bfloat162* w2 = reinterpret_cast<const __nv_bfloat162*>(&wv);
                    const __nv_bfloat162* u2 = reinterpret_cast<const __nv_bfloat162*>(&uv);
#pragma unroll
                    for (int q = 0; q < 4; ++q) {
                        const float w0 = __low2float(w2[q]), w1 = __high2float(w2[q]);
                        const float u0 = __low2float(u2[q]), u1 = __high2float(u2[q]);
#pragma unroll
                        for (int r = 0; r < GR_ROWS; ++r) {
                            const float a0 = As[r][kk + 2 * q], a1 = As[r][kk + 2 * q + 1];
                            acc[c][r] = fmaf(a1, w1, fmaf(a0, w0, acc[c][r]));
                            if (p.gated) accu[c][r] = fmaf(a1, u1, fmaf(a0, u0, accu[c][r]));
                        }
                    }
                }
                continue;
            }
            for (int kk = lane; kk < kc; kk += 32) {
                const float w = load_any(p.w, p.w_dt, wrow + kk);
                const float u = p.gated ? load_any(p.w, p.w_dt, urow + kk) : 0.f;
#pragma unroll
                for (int r = 0; r < GR_ROWS; ++r) {
                    acc[c][r] = fmaf(As[r][kk], w, acc[c][r]);
                    if (p.gated) accu[c][r] = fmaf(As[r][kk], u, accu[c][r]);
                }
            }
        }
    }
#pragma unroll
    for (int c = 0; c < CPW; ++c) {
        const int gn = n0 + warp * CPW + c;
#pragma unroll
        for (int r = 0; r < GR_ROWS; ++r) {
            const float g = warp_sum(acc[c][r]);
            const float u = p.gated ? warp_sum(accu[c][r]) : 0.f;
            const int pr = pair_of_row[r];
            if (lane == 0 && gn < p.N && pr >= 0)
                store_any(p.out, p.out_dt, (size_t)pr * p.out_stride + gn, p.gated ? silu_exact(g) * u : (p.relu2 ? relu_squared(g) : g));
        }
    }
}
}  // namespace

RS_EXPORT int rs_grouped_linear_rows_per_tile(int small) { return small ? GR_ROWS : GL_BM; }

RS_EXPORT int rs_grouped_linear(const void* a, int a_dt, long a_stride, int a_div, const void* w, int w_dt,
                                long w_expert_stride, void* out, int out_dt, long out_stride, const int* order,
                                const int* tiles, const int* n_tiles, int max_tiles, int N, int K, int gated, int small,
                                int relu2, void* stream) {
    if (max_tiles <= 0 || N <= 0) return 0;
    if (gated && relu2) return (int)cudaErrorInvalidValue;
    GroupedParams p{a, a_dt, a_stride, a_div, w, w_dt, w_expert_stride, out, out_dt, out_stride, order, tiles, n_tiles,
                    N, K, gated, relu2};
    cudaStream_t s = (cudaStream_t)stream;
    if (small) grouped_linear_rows_kernel<<<dim3((N + GR_COLS - 1) / GR_COLS, max_tiles), 256, 0, s>>>(p);
    else grouped_linear_tile_kernel<<<dim3((N + GL_BN - 1) / GL_BN, max_tiles), 256, 0, s>>>(p);
    return rs_launch_result();
}

// out[t, :] = weight * sum_k (pair_w[t * top + k] or 1) * pair_out[t * top + k, :] + sigmoid(h[t, :] . gate_w) * shared[t, :]
// (shared == null: no shared expert).  out is float32 [T, n].
__global__ void moe_combine_kernel(const float* __restrict__ pair_out, long pair_stride, int top, float weight,
                                   const float* __restrict__ pair_w,
                                   const void* __restrict__ shared, int shared_dt, long shared_stride,
                                   const void* __restrict__ h, int h_dt, long h_stride, const void* __restrict__ gate_w,
                                   int gate_dt, float* __restrict__ out, long out_stride, int n) {
    __shared__ float scratch[33];
    const int t = blockIdx.x;
    float gate = 0.f;
    if (shared != nullptr && gate_w != nullptr) {
        float d = 0.f;
        for (int i = threadIdx.x; i < n; i += blockDim.x)
            d = fmaf(load_any(h, h_dt, (size_t)t * h_stride + i), load_any(gate_w, gate_dt, i), d);
        d = block_sum(d, scratch);
        gate = 1.0f / (1.0f + expf(-d));
    } else if (shared != nullptr) {
        gate = 1.0f;
    }
    for (int i = threadIdx.x; i < n; i += blockDim.x) {
        float v = 0.f;
        if (pair_w != nullptr) {             // every pair with a weight of its own, k ascending
            for (int k = 0; k < top; ++k) v = fmaf(pair_w[(size_t)t * top + k], pair_out[(size_t)(t * top + k) * pair_stride + i], v);
        } else {
            for (int k = 0; k < top; ++k) v += pair_out[(size_t)(t * top + k) * pair_stride + i];
        }
        v *= weight;
        if (shared != nullptr) v = fmaf(gate, load_any(shared, shared_dt, (size_t)t * shared_stride + i), v);
        out[(size_t)t * out_stride + i] = v;
    }
}

RS_EXPORT int rs_moe_combine(const float* pair_out, long pair_stride, int top, float weight, const float* pair_w, const void* shared,
                             int shared_dt, long shared_stride, const void* h, int h_dt, long h_stride, const void* gate_w,
                             int gate_dt, float* out, long out_stride, int n_tokens, int n, void* stream) {
    if (n_tokens <= 0) return 0;
    moe_combine_kernel<<<n_tokens, 256, 0, (cudaStream_t)stream>>>(pair_out, pair_stride, top, weight, pair_w, shared, shared_dt,
                                                                  shared_stride, h, h_dt, h_stride, gate_w, gate_dt, out,
                                                                  out_stride, n);
    return rs_launch_result();
}
