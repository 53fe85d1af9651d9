// What surrounds attention whose queries, keys and values pass a short convolution over time, for both engines:
//   * conv_norm_kv_write: per channel of the projected [q | k | v] rows a causal convolution over time (the last
//     taps - 1 projected rows of every request come from its state slot), q and k heads divided by their root mean
//     square, q stored head by head in rows padded to the attention kernels' head size, k and v written into the
//     request's cache pages (padding zero);
//   * conv_tail_update: the state slot's last taps - 1 projected rows after the step;
//   * sigmoid_gate: joined heads times sigmoid(gate), out of the padded rows.
// The convolution, the norms and the sigmoid are float32; a (token, head) is a warp's, so its sums have one order.
#include "common.cuh"
#include <math.h>

namespace {
constexpr int MAX_PER_LANE = 8;          // head sizes up to 256

__device__ __forceinline__ void store_any(void* p, int dt, size_t i, float v) {
    if (dt == RS_F32) reinterpret_cast<float*>(p)[i] = v;
    else reinterpret_cast<__nv_bfloat16*>(p)[i] = __float2bfloat16_rn(v);
}

struct ConvKvParams {
    const void* proj; int dt; long proj_stride;       // [T, >= C] projected rows: q heads, then k heads, then v heads
    const void* w; int w_dt;                          // [taps, C] tap-major; null with taps == 0: no convolution
    const float* tail; long tail_stride;              // [slots, (taps - 1) * C]
    int C, taps;
    int n_q, n_kv, dk, dv, hdp;                       // head counts, key and value sizes, padded head size
    int unit_norm; float eps;
    void* q_out; long q_stride;                       // [T, n_q * hdp]
    void* cache; long page_stride; long v_offset;     // [pages][2][n_kv][page_size][hdp]
    int num_pages, page_size, write_kv;
    const int* block_table; int table_stride;
    const int* positions; int pos_stride; const int* seq_of_token; const int* q_start; const int* slots;
    int n_tokens;
    int* status;
};

// VEC neighbouring values starting at element i (a multiple of VEC when `vec`: one 4-, 8- or 16-byte access; else one by one)
template <int VEC>
__device__ __forceinline__ void load_run(const void* p, int dt, size_t i, bool vec, int n, float* v) {
    if (vec) {
        if (dt == RS_F32) {
            const float* f = reinterpret_cast<const float*>(p) + i;
            if constexpr (VEC == 1) { v[0] = f[0]; }
            else if constexpr (VEC == 2) { const float2 a = *reinterpret_cast<const float2*>(f); v[0] = a.x; v[1] = a.y; }
            else {
#pragma unroll
                for (int q = 0; q < VEC; q += 4) {
                    const float4 a = *reinterpret_cast<const float4*>(f + q);
                    v[q] = a.x; v[q + 1] = a.y; v[q + 2] = a.z; v[q + 3] = a.w;
                }
            }
        } else {
            const __nv_bfloat16* h = reinterpret_cast<const __nv_bfloat16*>(p) + i;
            if constexpr (VEC == 1) { v[0] = __bfloat162float(h[0]); }
            else if constexpr (VEC == 2) { const __nv_bfloat162 a = *reinterpret_cast<const __nv_bfloat162*>(h); v[0] = __low2float(a); v[1] = __high2float(a); }
            else if constexpr (VEC == 4) {
                const uint2 u = *reinterpret_cast<const uint2*>(h);
                const __nv_bfloat162* a = reinterpret_cast<const __nv_bfloat162*>(&u);
                v[0] = __low2float(a[0]); v[1] = __high2float(a[0]); v[2] = __low2float(a[1]); v[3] = __high2float(a[1]);
            } else {
                const uint4 u = *reinterpret_cast<const uint4*>(h);
                const __nv_bfloat162* a = reinterpret_cast<const __nv_bfloat162*>(&u);
#pragma unroll
                for (int q = 0; q < 4; ++q) { v[2 * q] = __low2float(a[q]); v[2 * q + 1] = __high2float(a[q]); }
            }
        }
    } else {
#pragma unroll
        for (int q = 0; q < VEC; ++q) v[q] = q < n ? load_any(p, dt, i + q) : 0.f;
    }
}

template <int VEC>
__device__ __forceinline__ void store_run(void* p, int dt, size_t i, bool vec, int n, const float* v) {
    if (vec && dt == RS_BF16 && VEC >= 2) {
        __nv_bfloat16* h = reinterpret_cast<__nv_bfloat16*>(p) + i;
        if constexpr (VEC == 2) { *reinterpret_cast<__nv_bfloat162*>(h) = __floats2bfloat162_rn(v[0], v[1]); }
        else if constexpr (VEC == 4) {
            uint2 u;
            __nv_bfloat162* a = reinterpret_cast<__nv_bfloat162*>(&u);
            a[0] = __floats2bfloat162_rn(v[0], v[1]); a[1] = __floats2bfloat162_rn(v[2], v[3]);
            *reinterpret_cast<uint2*>(h) = u;
        } else if constexpr (VEC == 8) {
            uint4 u;
            __nv_bfloat162* a = reinterpret_cast<__nv_bfloat162*>(&u);
#pragma unroll
            for (int q = 0; q < 4; ++q) a[q] = __floats2bfloat162_rn(v[2 * q], v[2 * q + 1]);
            *reinterpret_cast<uint4*>(h) = u;
        }
    } else {
#pragma unroll
        for (int q = 0; q < VEC; ++q) if (q < n) store_any(p, dt, i + q, v[q]);
    }
}

// A warp per (token, head); a lane owns VEC neighbouring channels of the head (32 * VEC >= the padded head size).  The
// warps of a CTA take neighbouring tokens of one head: the rows that the taps of one token read are the rows its
// neighbours read, so all but the first read of a row is served by the SM's own cache.
// which channels of a projected row head item `item` covers, and what it is (0 a query head, 1 a key head, 2 a value head)
__device__ __forceinline__ void item_span(const ConvKvParams& p, int item, int& base, int& width, int& kind) {
    if (item < p.n_q) { kind = 0; base = item * p.dk; width = p.dk; }
    else if (item < p.n_q + p.n_kv) { kind = 1; base = p.n_q * p.dk + (item - p.n_q) * p.dk; width = p.dk; }
    else { kind = 2; base = (p.n_q + p.n_kv) * p.dk + (item - p.n_q - p.n_kv) * p.dv; width = p.dv; }
}

// the warp's convolved head of token t (acc: this lane's VEC channels, zero beyond the head): unit norm, then to the
// query rows or the token's cache page, padding included
template <int VEC>
__device__ __forceinline__ void norm_and_store(const ConvKvParams& p, int vec_ok, int t, int s, int item, int kind, int width,
                                               int lane, float* acc) {
    const int d0 = lane * VEC;
    float r = 1.0f;
    if (p.unit_norm && kind != 2) {
        float ss = 0.f;
#pragma unroll
        for (int q = 0; q < VEC; ++q) ss = fmaf(acc[q], acc[q], ss);
        ss = warp_sum(ss);
        r = 1.0f / sqrtf(ss / (float)width + p.eps);
    }
    void* dst; size_t o;
    if (kind == 0) {
        dst = p.q_out; o = (size_t)t * p.q_stride + (size_t)item * p.hdp;
    } else {
        const int pos = p.positions[(size_t)t * p.pos_stride];
        const int page = p.block_table[(size_t)s * p.table_stride + pos / p.page_size];
        if (page < 0 || page >= p.num_pages) {
            if (lane == 0) atomicOr(p.status, RS_STATUS_BAD_PAGE);
            return;
        }
        const int g = kind == 1 ? item - p.n_q : item - p.n_q - p.n_kv;
        dst = p.cache;
        o = (size_t)page * p.page_stride + ((size_t)g * p.page_size + pos % p.page_size) * p.hdp + (kind == 2 ? p.v_offset : 0);
    }
#pragma unroll
    for (int q = 0; q < VEC; ++q) acc[q] *= r;
    const int n_out = min(max(p.hdp - d0, 0), VEC);    // the padding behind the head is written too (zeros)
    if (n_out > 0) store_run<VEC>(dst, p.dt, o + d0, vec_ok && n_out == VEC, n_out, acc);
}

// One (token, head) by a warp; a lane owns VEC neighbouring channels of the head (32 * VEC >= the padded head size).
// FAST: bfloat16 rows and weights with every run aligned (vec_ok): loads without run-time type or alignment branches, and
// for a token whose taps all read rows of this step, a loop the compiler can unroll with its loads issued together
// (one tap's load after the other's arithmetic made the kernel wait out the memory latency once per tap).
template <int VEC, bool FAST>
__device__ __forceinline__ void conv_one(const ConvKvParams& p, int vec_ok, int t, int item, int lane) {
    const int s = p.seq_of_token[t];
    const int row0 = p.q_start[s], li = t - row0;
    const float* tail = p.tail + (size_t)p.slots[s] * p.tail_stride;
    int base, width, kind;
    item_span(p, item, base, width, kind);
    const int d0 = lane * VEC;
    const int n = min(max(width - d0, 0), VEC);        // this lane's channels inside the head
    const bool vec = vec_ok && n == VEC;
    float acc[VEC];
#pragma unroll
    for (int q = 0; q < VEC; ++q) acc[q] = 0.f;
    if (n > 0) {
        const int c = base + d0;
        if (p.taps <= 0) {
            load_run<VEC>(p.proj, p.dt, (size_t)t * p.proj_stride + c, vec, n, acc);
        } else if (FAST && li >= p.taps - 1) {
            const size_t r0 = (size_t)(t - (p.taps - 1)) * p.proj_stride + c;
#pragma unroll 4
            for (int j = 0; j < p.taps; ++j) {
                float x[VEC], w[VEC];
                load_run<VEC>(p.proj, RS_BF16, r0 + (size_t)j * p.proj_stride, true, VEC, x);
                load_run<VEC>(p.w, RS_BF16, (size_t)j * p.C + c, true, VEC, w);
#pragma unroll
                for (int q = 0; q < VEC; ++q) acc[q] = fmaf(w[q], x[q], acc[q]);
            }
        } else {
            for (int j = 0; j < p.taps; ++j) {
                const int src = li - (p.taps - 1) + j;
                float x[VEC], w[VEC];
                if (src >= 0) load_run<VEC>(p.proj, p.dt, (size_t)(row0 + src) * p.proj_stride + c, vec, n, x);
                else load_run<VEC>(tail, RS_F32, (size_t)(p.taps - 1 + src) * p.C + c, vec, n, x);
                load_run<VEC>(p.w, p.w_dt, (size_t)j * p.C + c, vec, n, w);
#pragma unroll
                for (int q = 0; q < VEC; ++q) acc[q] = fmaf(w[q], x[q], acc[q]);
            }
        }
    }
    norm_and_store<VEC>(p, vec_ok, t, s, item, kind, width, lane, acc);
}

// The warps of a CTA take neighbouring tokens of one head.
template <int VEC, bool FAST>
__global__ void __launch_bounds__(256) conv_norm_kv_write_kernel(const ConvKvParams p, const int vec_ok) {
    const int lane = threadIdx.x & 31;
    const int items = p.n_q + (p.write_kv ? 2 * p.n_kv : 0);
    const unsigned wid = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);      // the launcher keeps tokens * items below 2^31
    if (wid >= (unsigned)p.n_tokens * (unsigned)items) return;
    const int item = (int)(wid / (unsigned)p.n_tokens), t = (int)(wid - (unsigned)item * (unsigned)p.n_tokens);
    conv_one<VEC, FAST>(p, vec_ok, t, item, lane);
}

// TPW neighbouring tokens of one head by a warp, for TAPS known at compile time and the FAST conditions: when the
// tokens belong to one sequence and none of their taps reaches before this step's rows, the warp loads the
// TAPS - 1 + TPW rows they read once, the head's weights once and the index arrays once; a tap's products are added
// in the order of the one-token form, so both forms give the same bits.  Any other group of tokens goes token by token.
template <int VEC, int TAPS, int TPW>
__global__ void __launch_bounds__(256) conv_norm_kv_write_multi_kernel(const ConvKvParams p) {
    const int lane = threadIdx.x & 31;
    const int items = p.n_q + (p.write_kv ? 2 * p.n_kv : 0);
    const unsigned groups = (unsigned)(p.n_tokens + TPW - 1) / TPW;
    const unsigned wid = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    if (wid >= groups * (unsigned)items) return;
    const int item = (int)(wid / groups), t0 = (int)(wid - (unsigned)item * groups) * TPW;
    const int nt = min(TPW, p.n_tokens - t0);
    const int s = p.seq_of_token[t0];
    const bool together = nt == TPW && p.seq_of_token[t0 + TPW - 1] == s && t0 - p.q_start[s] >= TAPS - 1;
    if (!together) {
        for (int tt = 0; tt < nt; ++tt) conv_one<VEC, true>(p, 1, t0 + tt, item, lane);
        return;
    }
    int base, width, kind;
    item_span(p, item, base, width, kind);
    const int d0 = lane * VEC;
    float acc[TPW][VEC];
#pragma unroll
    for (int tt = 0; tt < TPW; ++tt)
#pragma unroll
        for (int q = 0; q < VEC; ++q) acc[tt][q] = 0.f;
    if (width - d0 >= VEC) {                            // runs are whole under the FAST conditions
        const int c = base + d0;
        float w[TAPS][VEC];
#pragma unroll
        for (int j = 0; j < TAPS; ++j) load_run<VEC>(p.w, RS_BF16, (size_t)j * p.C + c, true, VEC, w[j]);
        const size_t r0 = (size_t)(t0 - (TAPS - 1)) * p.proj_stride + c;
#pragma unroll
        for (int r = 0; r < TAPS - 1 + TPW; ++r) {
            float x[VEC];
            load_run<VEC>(p.proj, RS_BF16, r0 + (size_t)r * p.proj_stride, true, VEC, x);
#pragma unroll
            for (int j = 0; j < TAPS; ++j) {
                const int tt = r - j;                   // row r is tap j of token tt
                if (tt >= 0 && tt < TPW) {
#pragma unroll
                    for (int q = 0; q < VEC; ++q) acc[tt][q] = fmaf(w[j][q], x[q], acc[tt][q]);
                }
            }
        }
    }
#pragma unroll
    for (int tt = 0; tt < TPW; ++tt) norm_and_store<VEC>(p, 1, t0 + tt, s, item, kind, width, lane, acc[tt]);
}

// tail[i] <- the projected row at local index q_len - (taps - 1) + i: a row of this step, or a row the tail held.
// One thread per (sequence, channel), i ascending: a row read from the tail lies behind the one being written.
__global__ void conv_tail_update_kernel(const void* __restrict__ proj, int dt, long proj_stride, float* __restrict__ tails,
                                        long tail_stride, const int* __restrict__ q_start, const int* __restrict__ slots,
                                        int C, int taps, int n_seqs) {
    const long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= (long)n_seqs * C) return;
    const int s = (int)(idx / C), c = (int)(idx % C);
    const int row0 = q_start[s], q_len = q_start[s + 1] - row0;
    float* tail = tails + (size_t)slots[s] * tail_stride;
    for (int i = 0; i < taps - 1; ++i) {
        const int src = q_len - (taps - 1) + i;
        tail[(size_t)i * C + c] = src >= 0 ? load_any(proj, dt, (size_t)(row0 + src) * proj_stride + c)
                                           : tail[(size_t)(taps - 1 + src) * C + c];
    }
}

// out[t, h * dv + d] = a[t, h * hdp + d] * sigmoid(g[t, h * dv + d])    (g == null: a copy out of the padded rows)
// A thread takes VEC neighbouring values of one head (dv a multiple of VEC, every row and head aligned for it).
template <int VEC>
__global__ void sigmoid_gate_kernel(const void* __restrict__ a, long a_stride, const void* __restrict__ g, long g_stride,
                                    void* __restrict__ out, long out_stride, int dt, int n_heads, int dv, int hdp,
                                    int n_tokens) {
    const long idx = (long)blockIdx.x * blockDim.x + threadIdx.x;
    const int W = n_heads * dv / VEC;
    if (idx >= (long)n_tokens * W) return;
    const int t = (int)(idx / W), c = (int)(idx % W) * VEC;
    const int h = c / dv, d = c % dv;
    float v[VEC], z[VEC];
    load_run<VEC>(a, dt, (size_t)t * a_stride + (size_t)h * hdp + d, true, VEC, v);
    if (g != nullptr) {
        load_run<VEC>(g, dt, (size_t)t * g_stride + c, true, VEC, z);
#pragma unroll
        for (int q = 0; q < VEC; ++q) v[q] *= 1.0f / (1.0f + expf(-z[q]));
    }
    store_run<VEC>(out, dt, (size_t)t * out_stride + c, true, VEC, v);
}
}  // namespace

RS_EXPORT int rs_conv_norm_kv_write(const void* proj, int dt, long proj_stride, const void* w, int w_dt, float* tails,
                                    long tail_stride, int C, int taps, int n_q, int n_kv, int dk, int dv, int hdp,
                                    int unit_norm, float eps, void* q_out, long q_stride, void* cache, long page_stride,
                                    int num_pages, int page_size, int write_kv, const int* block_table, int table_stride,
                                    const int* positions, int pos_stride, const int* seq_of_token, const int* q_start,
                                    const int* slots, int n_tokens, int n_seqs, int* status, void* stream) {
    if (n_tokens <= 0) return 0;
    if (hdp > 32 * MAX_PER_LANE || dk > hdp || dv > hdp || dk <= 0 || dv <= 0 || (taps > 0 && w == nullptr) ||
        (taps > 1 && tails == nullptr))
        return (int)cudaErrorInvalidValue;
    ConvKvParams p{proj, dt, proj_stride, w, w_dt, tails, tail_stride, C, taps, n_q, n_kv, dk, dv, hdp, unit_norm, eps,
                   q_out, q_stride, cache, page_stride, (long)n_kv * page_size * hdp, num_pages, page_size, write_kv,
                   block_table, table_stride, positions, pos_stride, seq_of_token, q_start, slots, n_tokens, status};
    cudaStream_t s = (cudaStream_t)stream;
    const long warps = (long)n_tokens * (n_q + (write_kv ? 2 * n_kv : 0));
    if (warps >= (1L << 31)) return (int)cudaErrorInvalidValue;
    const unsigned blocks = (unsigned)((warps + 7) / 8);
    const int vec_n = hdp <= 32 ? 1 : (hdp <= 64 ? 2 : (hdp <= 128 ? 4 : 8));
    // vector accesses: every run of a lane starts at a multiple of its length, in every array it touches
    const int es = dt == RS_F32 ? 4 : 2;
    const bool vec_ok = dk % vec_n == 0 && dv % vec_n == 0 && hdp % vec_n == 0 && proj_stride % vec_n == 0 && C % vec_n == 0 &&
                        q_stride % vec_n == 0 && tail_stride % vec_n == 0 && page_stride % vec_n == 0 &&
                        ((size_t)proj % (vec_n * es)) == 0 && ((size_t)q_out % (vec_n * es)) == 0 &&
                        ((size_t)cache % (vec_n * es)) == 0 && ((size_t)tails % (vec_n * 4)) == 0 &&
                        ((size_t)w % (vec_n * (w_dt == RS_F32 ? 4 : 2))) == 0;
    const bool fast = vec_ok && dt == RS_BF16 && (taps <= 0 || w_dt == RS_BF16);
    constexpr int TPW = 4;
    // several tokens a warp where the step is mostly portions; a step of single tokens keeps a warp per token
    if (fast && taps >= 2 && taps <= 4 && n_tokens >= 2 * TPW * n_seqs) {
        const long groups = (n_tokens + TPW - 1) / TPW;
        const unsigned mblocks = (unsigned)((groups * (n_q + (write_kv ? 2 * n_kv : 0)) + 7) / 8);
#define RS_CONV_MULTI(V)                                                                                   \
        do {                                                                                               \
            if (taps == 2) conv_norm_kv_write_multi_kernel<V, 2, TPW><<<mblocks, 256, 0, s>>>(p);          \
            else if (taps == 3) conv_norm_kv_write_multi_kernel<V, 3, TPW><<<mblocks, 256, 0, s>>>(p);     \
            else conv_norm_kv_write_multi_kernel<V, 4, TPW><<<mblocks, 256, 0, s>>>(p);                    \
        } while (0)
        if (vec_n == 1) RS_CONV_MULTI(1);
        else if (vec_n == 2) RS_CONV_MULTI(2);
        else if (vec_n == 4) RS_CONV_MULTI(4);
        else RS_CONV_MULTI(8);
#undef RS_CONV_MULTI
    } else if (fast) {
        if (vec_n == 1) conv_norm_kv_write_kernel<1, true><<<blocks, 256, 0, s>>>(p, vec_ok);
        else if (vec_n == 2) conv_norm_kv_write_kernel<2, true><<<blocks, 256, 0, s>>>(p, vec_ok);
        else if (vec_n == 4) conv_norm_kv_write_kernel<4, true><<<blocks, 256, 0, s>>>(p, vec_ok);
        else conv_norm_kv_write_kernel<8, true><<<blocks, 256, 0, s>>>(p, vec_ok);
    } else {
        if (vec_n == 1) conv_norm_kv_write_kernel<1, false><<<blocks, 256, 0, s>>>(p, vec_ok);
        else if (vec_n == 2) conv_norm_kv_write_kernel<2, false><<<blocks, 256, 0, s>>>(p, vec_ok);
        else if (vec_n == 4) conv_norm_kv_write_kernel<4, false><<<blocks, 256, 0, s>>>(p, vec_ok);
        else conv_norm_kv_write_kernel<8, false><<<blocks, 256, 0, s>>>(p, vec_ok);
    }
    int e = rs_launch_result();
    if (e != 0 || taps <= 1) return e;
    const long n = (long)n_seqs * C;
    conv_tail_update_kernel<<<(unsigned)((n + 255) / 256), 256, 0, s>>>(proj, dt, proj_stride, tails, tail_stride, q_start,
                                                                         slots, C, taps, n_seqs);
    return rs_launch_result();
}

RS_EXPORT int rs_sigmoid_gate(const void* a, long a_stride, const void* g, long g_stride, void* out, long out_stride, int dt,
                              int n_heads, int dv, int hdp, int n_tokens, void* stream) {
    if (n_tokens <= 0) return 0;
    const long n = (long)n_tokens * n_heads * dv;
    const int es = dt == RS_F32 ? 4 : 2;
    const bool vec8 = dv % 8 == 0 && hdp % 8 == 0 && a_stride % 8 == 0 && g_stride % 8 == 0 && out_stride % 8 == 0 &&
                      ((size_t)a % (8 * es)) == 0 && ((size_t)g % (8 * es)) == 0 && ((size_t)out % (8 * es)) == 0;
    cudaStream_t s = (cudaStream_t)stream;
    if (vec8) sigmoid_gate_kernel<8><<<(unsigned)((n / 8 + 255) / 256), 256, 0, s>>>(a, a_stride, g, g_stride, out, out_stride,
                                                                                   dt, n_heads, dv, hdp, n_tokens);
    else sigmoid_gate_kernel<1><<<(unsigned)((n + 255) / 256), 256, 0, s>>>(a, a_stride, g, g_stride, out, out_stride, dt,
                                                                          n_heads, dv, hdp, n_tokens);
    return rs_launch_result();
}
