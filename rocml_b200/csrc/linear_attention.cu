// Linear attention with a fixed decay per head: a running sum instead of a softmax over all keys.
//
//   S_t = d_h * S_(t-1) + k_t v_t^T          S [dim, vdim] per (sequence, head), 32-bit, zero at the start
//   o_t = S_t^T q_t
//
// q, k, v are columns of the layer's stacked projection (in the activations' type, or as 32-bit partial
// sums over K that are added first, in order), optionally through silu, k times a constant.  Everything that
// enters the recurrence from there on is 32-bit: the decay, the state, the sums.
//
//   decay_scan    a block owns one (sequence, head) and a tile of the state's columns (columns are independent of
//                 one another); the tile lives in shared memory for the whole step and goes back to the
//                 sequence's slot at the end.  Tokens are taken eight at a time: their q, k, v are staged once,
//                 then every thread walks the eight tokens over its own part of a column (rows i = p, p + P, ..),
//                 so no barrier separates tokens; the parts' sums meet in shared memory and are added in the
//                 order of p.  One token a sequence (a decode step) is the same kernel with one token.
//                 The order of a token's operations does not depend on how the prompt was cut or on the batch.
//   group_norm_gate   what follows the recurrence: o divided by its root mean square over each of G groups of
//                 columns (G = heads: per head; G = 1: all heads together), times an optional weight vector, times
//                 act(gate) with the gate another column block of the projection; written in the activations' type
//                 for the output product.
#include "common.cuh"
#include "api.h"

using namespace rb;

namespace {
constexpr int SCAN_THREADS = 256;
constexpr int SCAN_TB = 8;          // tokens staged at a time

template <typename IT>
__device__ __forceinline__ float load_sum(const IT* p, int n_in, size_t in_stride) {
    float v = 0.f;
    for (int s = 0; s < n_in; ++s) v += to_f32(p[(size_t)s * in_stride]);
    return v;
}

template <typename IT>
__global__ void __launch_bounds__(SCAN_THREADS)
decay_scan_kernel(const IT* __restrict__ in, int n_in, size_t in_stride, int row_stride, int q_off, int k_off, int v_off,
                  int heads, int dim, int vdim, int act_qk, int act_v, float k_scale, const float* __restrict__ decay,
                  float* __restrict__ state, const int* __restrict__ seq_slot, const int* __restrict__ cu_q,
                  float* __restrict__ out, int ld_out, int VT, int P) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ __align__(16) float sm[];
    float* S = sm;                              // [dim][VT]
    float* qs = S + (size_t)dim * VT;           // [TB][dim]
    float* ks = qs + SCAN_TB * dim;             // [TB][dim]
    float* vs = ks + SCAN_TB * dim;             // [TB][VT]
    float* part = vs + SCAN_TB * VT;            // [TB][P][VT]
    const int b = blockIdx.z, h = blockIdx.y, v0 = blockIdx.x * VT;
    const int slot = seq_slot[b];
    if (slot < 0) return;
    const int t_begin = cu_q[b], t_end = cu_q[b + 1];
    if (t_end <= t_begin) return;
    const int vt = min(VT, vdim - v0);
    const int tid = threadIdx.x;
    const float d = decay[h];
    float* st = state + (((size_t)slot * heads + h) * dim) * vdim + v0;
    for (int idx = tid; idx < dim * VT; idx += SCAN_THREADS) {
        const int i = idx / VT, j = idx - i * VT;
        S[idx] = j < vt ? st[(size_t)i * vdim + j] : 0.f;
    }
    const int p = tid / VT, j = tid - p * VT;   // this thread's part of column j
    const bool works = p < P && j < vt;
    for (int t0 = t_begin; t0 < t_end; t0 += SCAN_TB) {
        const int nb = min(SCAN_TB, t_end - t0);
        for (int idx = tid; idx < nb * dim; idx += SCAN_THREADS) {
            const int tt = idx / dim, i = idx - tt * dim;
            const IT* row = in + (size_t)(t0 + tt) * row_stride + (size_t)h * dim + i;
            float q = load_sum(row + q_off, n_in, in_stride), k = load_sum(row + k_off, n_in, in_stride);
            if (act_qk == 1) { q = silu(q); k = silu(k); }
            qs[idx] = q;
            ks[idx] = k * k_scale;
        }
        for (int idx = tid; idx < nb * VT; idx += SCAN_THREADS) {
            const int tt = idx / VT, jj = idx - tt * VT;
            float v = 0.f;
            if (jj < vt) {
                v = load_sum(in + (size_t)(t0 + tt) * row_stride + v_off + (size_t)h * vdim + v0 + jj, n_in, in_stride);
                if (act_v == 1) v = silu(v);
            }
            vs[idx] = v;
        }
        __syncthreads();
        if (works) {
            for (int tt = 0; tt < nb; ++tt) {
                const float v = vs[tt * VT + j];
                const float* q = qs + tt * dim;
                const float* k = ks + tt * dim;
                float acc = 0.f;
                for (int i = p; i < dim; i += P) {
                    const float s = fmaf(k[i], v, d * S[i * VT + j]);
                    S[i * VT + j] = s;
                    acc = fmaf(s, q[i], acc);
                }
                part[(tt * P + p) * VT + j] = acc;
            }
        }
        __syncthreads();
        for (int idx = tid; idx < nb * VT; idx += SCAN_THREADS) {
            const int tt = idx / VT, jj = idx - tt * VT;
            if (jj >= vt) continue;
            float o = 0.f;
            for (int pp = 0; pp < P; ++pp) o += part[(tt * P + pp) * VT + jj];
            out[(size_t)(t0 + tt) * ld_out + (size_t)h * vdim + v0 + jj] = o;
        }
    }
    __syncthreads();
    for (int idx = tid; idx < dim * VT; idx += SCAN_THREADS) {
        const int i = idx / VT, jj = idx - i * VT;
        if (jj < vt) st[(size_t)i * vdim + jj] = S[idx];
    }
}

// ---- one token a sequence: the state streams through registers -----------------------------------------------------
// A block owns a (sequence, head) and 32 of the state's columns; a warp takes every eighth row, a lane a column, so a
// row's 32 entries are one 128-byte access and nothing of the state passes through shared memory.  Every entry is read,
// decayed, updated and written once; the warps' sums over their rows meet in shared memory and are added in the
// order of the warps.
template <typename IT>
__global__ void __launch_bounds__(256)
decay_step_kernel(const IT* __restrict__ in, int n_in, size_t in_stride, int row_stride, int q_off, int k_off, int v_off,
                  int heads, int dim, int vdim, int act_qk, int act_v, float k_scale, const float* __restrict__ decay,
                  float* __restrict__ state, const int* __restrict__ seq_slot, const int* __restrict__ cu_q,
                  float* __restrict__ out, int ld_out) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ __align__(16) float sm[];
    __shared__ float part[8][32];
    float* qs = sm;            // [dim]
    float* ks = sm + dim;      // [dim]
    const int b = blockIdx.z, h = blockIdx.y;
    const int slot = seq_slot[b];
    if (slot < 0) return;
    const int t = cu_q[b];
    if (cu_q[b + 1] <= t) return;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int j = blockIdx.x * 32 + lane;
    const IT* row = in + (size_t)t * row_stride;
    for (int i = threadIdx.x; i < dim; i += 256) {
        float q = load_sum(row + q_off + h * dim + i, n_in, in_stride), k = load_sum(row + k_off + h * dim + i, n_in, in_stride);
        if (act_qk == 1) { q = silu(q); k = silu(k); }
        qs[i] = q;
        ks[i] = k * k_scale;
    }
    float v = 0.f;
    if (j < vdim) {
        v = load_sum(row + v_off + h * vdim + j, n_in, in_stride);
        if (act_v == 1) v = silu(v);
    }
    __syncthreads();
    const float d = decay[h];
    float* S = state + (((size_t)slot * heads + h) * dim) * vdim + j;
    float acc = 0.f;
    if (j < vdim) {
        int i = warp;
        for (; i + 24 < dim; i += 32) {           // four rows' loads in flight
            float s0 = S[(size_t)i * vdim], s1 = S[(size_t)(i + 8) * vdim], s2 = S[(size_t)(i + 16) * vdim], s3 = S[(size_t)(i + 24) * vdim];
            s0 = fmaf(ks[i], v, d * s0); s1 = fmaf(ks[i + 8], v, d * s1); s2 = fmaf(ks[i + 16], v, d * s2); s3 = fmaf(ks[i + 24], v, d * s3);
            S[(size_t)i * vdim] = s0; S[(size_t)(i + 8) * vdim] = s1; S[(size_t)(i + 16) * vdim] = s2; S[(size_t)(i + 24) * vdim] = s3;
            acc = fmaf(s0, qs[i], acc); acc = fmaf(s1, qs[i + 8], acc); acc = fmaf(s2, qs[i + 16], acc); acc = fmaf(s3, qs[i + 24], acc);
        }
        for (; i < dim; i += 8) {
            const float s = fmaf(ks[i], v, d * S[(size_t)i * vdim]);
            S[(size_t)i * vdim] = s;
            acc = fmaf(s, qs[i], acc);
        }
    }
    part[warp][lane] = acc;
    __syncthreads();
    if (warp == 0 && j < vdim) {
        float o = 0.f;
#pragma unroll
        for (int w = 0; w < 8; ++w) o += part[w][lane];
        out[(size_t)t * ld_out + (size_t)h * vdim + j] = o;
    }
}

// ---- prompts: the same sums by blocks of 64 tokens, all blocks at once ----------------------------------------------
// Within a block of m tokens that starts from the state S0:
//   o_t   = d^(t+1) S0^T q_t + sum_{s <= t} d^(t-s) (q_t . k_s) v_s           t = 0 .. m-1
//   S_end = d^m S0 + sum_s d^(m-1-s) k_s v_s^T
// Three kernels: (1) every block's own sum L = sum_s d^(m-1-s) k_s v_s^T; (2) along each sequence, S0 of every block
// from the slot's state and the L's before it (the L's place receives S0; the slot receives the last S_end);
// (3) every block's outputs.  A block of the grid finds its (sequence, block of tokens) from cu_q.  All 32-bit FMA.
constexpr int CB = 64;              // tokens a block
constexpr int CT = 256;             // threads

__device__ __forceinline__ float decay_pow(float d, int n) {
    float r = 1.f, b = d;
    while (n > 0) { if (n & 1) r *= b; b *= b; n >>= 1; }
    return r;
}

// Which sequence and which of its blocks of tokens the grid's block `g` is: blocks are numbered sequence after
// sequence.  Returns false when g lies past the last one.  t0, m: the block's first row and its rows; first: the number
// of the sequence's first block; slot: the sequence's slot (-1: padding).
__device__ __forceinline__ bool find_block(int g, const int* seq_slot, const int* cu_q, int B, int* b_out, int* t0, int* m,
                                           int* first, int* slot) {
    int base = 0;
    for (int b = 0; b < B; ++b) {
        const int n = cu_q[b + 1] - cu_q[b];
        const int nb = seq_slot[b] >= 0 ? (n + CB - 1) / CB : 0;
        if (g < base + nb) {
            const int c = g - base;
            *b_out = b; *t0 = cu_q[b] + c * CB; *m = min(CB, n - c * CB); *first = base; *slot = seq_slot[b];
            return true;
        }
        base += nb;
    }
    return false;
}

// m rows of `width` columns from column col0 of the projection rows into shared memory as 32-bit numbers (partial sums
// added, the activation applied, times factor and the row's own factor); TR: transposed, dst[column][row].  16 bytes a
// load where the columns and strides allow.
template <typename IT, bool TR>
__device__ __forceinline__ void stage_rows(const IT* in, int n_in, size_t in_stride, int row_stride, int t0, int m, int col0,
                                           int width, int act, float* dst, int ld, const float* row_factor, float factor) {
    constexpr int V = sizeof(IT) == 2 ? 8 : 4;
    const bool vec = width % V == 0 && row_stride % V == 0 && col0 % V == 0 && in_stride % V == 0 && ((uintptr_t)in & 15) == 0;
    if (vec) {
        const int wv = width / V;
        for (int idx = threadIdx.x; idx < m * wv; idx += CT) {
            const int tt = idx / wv, i0 = (idx - tt * wv) * V;
            const IT* p = in + (size_t)(t0 + tt) * row_stride + col0 + i0;
            float x[V];
#pragma unroll
            for (int u = 0; u < V; ++u) x[u] = 0.f;
            for (int s = 0; s < n_in; ++s) {
                const uint4 raw = *reinterpret_cast<const uint4*>(p + (size_t)s * in_stride);
                if (sizeof(IT) == 2) {
                    const uint32_t w[4] = {raw.x, raw.y, raw.z, raw.w};
#pragma unroll
                    for (int u = 0; u < 4; ++u) {
                        x[2 * u] += __uint_as_float(w[u] << 16);
                        x[2 * u + 1] += __uint_as_float(w[u] & 0xFFFF0000u);
                    }
                } else {
                    x[0] += __uint_as_float(raw.x); x[1] += __uint_as_float(raw.y);
                    x[2] += __uint_as_float(raw.z); x[3] += __uint_as_float(raw.w);
                }
            }
            const float f = factor * (row_factor ? row_factor[tt] : 1.f);
#pragma unroll
            for (int u = 0; u < V; ++u) {
                float y = x[u];
                if (act == 1) y = silu(y);
                if (TR) dst[(i0 + u) * ld + tt] = y * f;
                else dst[tt * ld + i0 + u] = y * f;
            }
        }
        return;
    }
    for (int idx = threadIdx.x; idx < m * width; idx += CT) {
        const int tt = idx / width, i = idx - tt * width;
        float x = load_sum(in + (size_t)(t0 + tt) * row_stride + col0 + i, n_in, in_stride);
        if (act == 1) x = silu(x);
        x *= factor * (row_factor ? row_factor[tt] : 1.f);
        if (TR) dst[i * ld + tt] = x;
        else dst[tt * ld + i] = x;
    }
}

template <typename IT, int R>
__global__ void __launch_bounds__(CT, 2)
chunk_state_kernel(const IT* __restrict__ in, int n_in, size_t in_stride, int row_stride, int k_off, int v_off, int heads,
                   int dim, int vdim, int act_qk, int act_v, float k_scale, const float* __restrict__ decay,
                   const int* __restrict__ seq_slot, const int* __restrict__ cu_q, int B, float* __restrict__ Lbuf) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ __align__(16) float sm[];
    __shared__ float pw[CB + 1];
    int b, t0, m, first, slot;
    if (!find_block(blockIdx.x, seq_slot, cu_q, B, &b, &t0, &m, &first, &slot)) return;
    const int h = blockIdx.y;
    const float d = decay[h];
    float* ks = sm;                       // [m][dim], row s already times d^(m-1-s)
    float* vs = ks + CB * dim;            // [m][vdim]
    if (threadIdx.x < m) pw[threadIdx.x] = decay_pow(d, m - 1 - threadIdx.x);
    __syncthreads();
    stage_rows<IT, false>(in, n_in, in_stride, row_stride, t0, m, k_off + h * dim, dim, act_qk, ks, dim, pw, k_scale);
    stage_rows<IT, false>(in, n_in, in_stride, row_stride, t0, m, v_off + h * vdim, vdim, act_v, vs, vdim, nullptr, 1.f);
    __syncthreads();
    const int ty = threadIdx.x >> 4, tx = threadIdx.x & 15;
    float acc[R][R];
#pragma unroll
    for (int a = 0; a < R; ++a)
#pragma unroll
        for (int c = 0; c < R; ++c) acc[a][c] = 0.f;
    for (int s = 0; s < m; ++s) {
        float kk[R], vv[R];
#pragma unroll
        for (int a = 0; a < R; ++a) kk[a] = ty + 16 * a < dim ? ks[s * dim + ty + 16 * a] : 0.f;
#pragma unroll
        for (int c = 0; c < R; ++c) vv[c] = tx + 16 * c < vdim ? vs[s * vdim + tx + 16 * c] : 0.f;
#pragma unroll
        for (int a = 0; a < R; ++a)
#pragma unroll
            for (int c = 0; c < R; ++c) acc[a][c] = fmaf(kk[a], vv[c], acc[a][c]);
    }
    float* L = Lbuf + ((size_t)blockIdx.x * heads + h) * dim * vdim;
#pragma unroll
    for (int a = 0; a < R; ++a)
#pragma unroll
        for (int c = 0; c < R; ++c)
            if (ty + 16 * a < dim && tx + 16 * c < vdim) L[(size_t)(ty + 16 * a) * vdim + tx + 16 * c] = acc[a][c];
}

// A thread owns V neighbouring entries of the state (V = 4 where the state's size allows 16-byte accesses) and walks the
// sequence's blocks in order; the loads of eight blocks are in flight together (they do not depend on the running
// state), so the walk is not one memory latency a block.
template <int V>
__global__ void __launch_bounds__(256)
chunk_prefix_kernel(const float* __restrict__ decay, float* __restrict__ state, const int* __restrict__ seq_slot,
                    const int* __restrict__ cu_q, int B, int heads, int dim, int vdim, float* __restrict__ Lbuf) {
    pdl_trigger();
    pdl_wait();
    const int b = blockIdx.z, h = blockIdx.y;
    const int slot = seq_slot[b];
    if (slot < 0) return;
    const int n = cu_q[b + 1] - cu_q[b];
    if (n <= 0) return;
    int first = 0;
    for (int i = 0; i < b; ++i)
        if (seq_slot[i] >= 0) first += (cu_q[i + 1] - cu_q[i] + CB - 1) / CB;
    const int e = (blockIdx.x * blockDim.x + threadIdx.x) * V;
    if (e >= dim * vdim) return;
    const float d = decay[h];
    const float d_full = decay_pow(d, CB);
    struct alignas(4 * V) Vec { float x[V]; };
    const size_t sz = (size_t)dim * vdim;
    Vec* st = reinterpret_cast<Vec*>(state + ((size_t)slot * heads + h) * sz + e);
    Vec run = *st;
    const int nb = (n + CB - 1) / CB;
    constexpr int U = 8;
    for (int c0 = 0; c0 < nb; c0 += U) {
        Vec own[U];
#pragma unroll
        for (int u = 0; u < U; ++u)
            if (c0 + u < nb) own[u] = *reinterpret_cast<const Vec*>(Lbuf + ((size_t)(first + c0 + u) * heads + h) * sz + e);
#pragma unroll
        for (int u = 0; u < U; ++u) {
            if (c0 + u >= nb) break;
            *reinterpret_cast<Vec*>(Lbuf + ((size_t)(first + c0 + u) * heads + h) * sz + e) = run;   // what this block starts from
            const int m = min(CB, n - (c0 + u) * CB);
            const float f = m == CB ? d_full : decay_pow(d, m);
#pragma unroll
            for (int v = 0; v < V; ++v) run.x[v] = fmaf(f, run.x[v], own[u].x[v]);
        }
    }
    *st = run;
}

template <typename IT, int R>
__global__ void __launch_bounds__(CT, 2)
chunk_out_kernel(const IT* __restrict__ in, int n_in, size_t in_stride, int row_stride, int q_off, int k_off, int v_off,
                 int heads, int dim, int vdim, int act_qk, int act_v, float k_scale, const float* __restrict__ decay,
                 const int* __restrict__ seq_slot, const int* __restrict__ cu_q, int B, const float* __restrict__ Lbuf,
                 float* __restrict__ out, int ld_out) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ __align__(16) float sm[];
    __shared__ float pw[CB + 1];
    int b, t0, m, first, slot;
    if (!find_block(blockIdx.x, seq_slot, cu_q, B, &b, &t0, &m, &first, &slot)) return;
    const int h = blockIdx.y;
    const float d = decay[h];
    // No padding anywhere (two blocks then fit a multiprocessor at head size 128): a warp reads two rows of q and of
    // A at one column (broadcasts), and 16 neighbouring entries of a row of k^T, v or the state.
    const int ldq = dim;
    float* qs = sm;                        // [CB][dim]
    float* ks = qs + CB * dim;             // k transposed, [dim][CB]; later slabs of the starting state
    float* vs = ks + CB * dim;             // [CB][vdim]
    float* A = vs + CB * vdim;             // [CB][CB]
    if (threadIdx.x <= CB) pw[threadIdx.x] = decay_pow(d, threadIdx.x);
    stage_rows<IT, false>(in, n_in, in_stride, row_stride, t0, m, q_off + h * dim, dim, act_qk, qs, ldq, nullptr, 1.f);
    stage_rows<IT, true>(in, n_in, in_stride, row_stride, t0, m, k_off + h * dim, dim, act_qk, ks, CB, nullptr, k_scale);
    stage_rows<IT, false>(in, n_in, in_stride, row_stride, t0, m, v_off + h * vdim, vdim, act_v, vs, vdim, nullptr, 1.f);
    __syncthreads();
    const int ty = threadIdx.x >> 4, tx = threadIdx.x & 15;
    {
        // A[t][s] = d^(t-s) (q_t . k_s) for s <= t, else 0: t = ty + 16 a, s = tx + 16 c
        float acc[4][4];
#pragma unroll
        for (int a = 0; a < 4; ++a)
#pragma unroll
            for (int c = 0; c < 4; ++c) acc[a][c] = 0.f;
        for (int i = 0; i < dim; ++i) {
            float qq[4], kk[4];
#pragma unroll
            for (int a = 0; a < 4; ++a) qq[a] = ty + 16 * a < m ? qs[(ty + 16 * a) * ldq + i] : 0.f;
#pragma unroll
            for (int c = 0; c < 4; ++c) kk[c] = tx + 16 * c < m ? ks[i * CB + tx + 16 * c] : 0.f;
#pragma unroll
            for (int a = 0; a < 4; ++a)
#pragma unroll
                for (int c = 0; c < 4; ++c) acc[a][c] = fmaf(qq[a], kk[c], acc[a][c]);
        }
#pragma unroll
        for (int a = 0; a < 4; ++a)
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const int t = ty + 16 * a, s = tx + 16 * c;
                A[t * CB + s] = (s <= t && t < m) ? acc[a][c] * pw[t - s] : 0.f;
            }
    }
    __syncthreads();
    // o[t][j]: t = ty + 16 a (a < 4), j = tx + 16 c (c < R)
    float o1[4][R], o2[4][R];
#pragma unroll
    for (int a = 0; a < 4; ++a)
#pragma unroll
        for (int c = 0; c < R; ++c) { o1[a][c] = 0.f; o2[a][c] = 0.f; }
    for (int s = 0; s < m; ++s) {
        float aa[4], vv[R];
#pragma unroll
        for (int a = 0; a < 4; ++a) aa[a] = A[(ty + 16 * a) * CB + s];
#pragma unroll
        for (int c = 0; c < R; ++c) vv[c] = tx + 16 * c < vdim ? vs[s * vdim + tx + 16 * c] : 0.f;
#pragma unroll
        for (int a = 0; a < 4; ++a)
#pragma unroll
            for (int c = 0; c < R; ++c) o1[a][c] = fmaf(aa[a], vv[c], o1[a][c]);
    }
    // the part that comes from before the block: slabs of 32 rows of the starting state go through ks
    const float* S0 = Lbuf + ((size_t)blockIdx.x * heads + h) * dim * vdim;
    for (int i0 = 0; i0 < dim; i0 += 32) {
        __syncthreads();
        const int rows = min(32, dim - i0);
        for (int idx = threadIdx.x; idx < rows * vdim; idx += CT) ks[idx] = S0[(size_t)i0 * vdim + idx];
        __syncthreads();
        for (int i = 0; i < rows; ++i) {
            float qq[4], ss[R];
#pragma unroll
            for (int a = 0; a < 4; ++a) qq[a] = ty + 16 * a < m ? qs[(ty + 16 * a) * ldq + i0 + i] : 0.f;
#pragma unroll
            for (int c = 0; c < R; ++c) ss[c] = tx + 16 * c < vdim ? ks[i * vdim + tx + 16 * c] : 0.f;
#pragma unroll
            for (int a = 0; a < 4; ++a)
#pragma unroll
                for (int c = 0; c < R; ++c) o2[a][c] = fmaf(qq[a], ss[c], o2[a][c]);
        }
    }
#pragma unroll
    for (int a = 0; a < 4; ++a) {
        const int t = ty + 16 * a;
        if (t >= m) continue;
        const float f = pw[t + 1];
#pragma unroll
        for (int c = 0; c < R; ++c)
            if (tx + 16 * c < vdim) out[(size_t)(t0 + t) * ld_out + (size_t)h * vdim + tx + 16 * c] = fmaf(f, o2[a][c], o1[a][c]);
    }
}

// One block a token.  in: o float32 [T, W]; gate: columns g_off .. g_off + W of the projection rows.
template <typename IT, typename AT, typename WT>
__global__ void __launch_bounds__(256)
group_norm_gate_kernel(const float* __restrict__ o, int ld_o, const IT* __restrict__ proj, int n_in, size_t in_stride,
                       int row_stride, int g_off, const WT* __restrict__ w, float eps, int groups, int W, int gate_act,
                       AT* __restrict__ out, int ld_out, const int* __restrict__ slot_of_token) {
    pdl_trigger();
    pdl_wait();
    __shared__ float scratch[33];
    const int t = blockIdx.x;
    if (slot_of_token[t] < 0) return;
    const float* row = o + (size_t)t * ld_o;
    const IT* g = proj + (size_t)t * row_stride + g_off;
    AT* dst = out + (size_t)t * ld_out;
    const int gw = W / groups;
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nwarps = blockDim.x >> 5;
    // four columns a thread where sizes and addresses allow: a warp a group (or the whole block the one group)
    if ((gw & 3) == 0 && (ld_o & 3) == 0 && (row_stride & 3) == 0 && (g_off & 3) == 0 && (in_stride & 3) == 0 && (ld_out & 3) == 0 &&
        ((uintptr_t)o & 15) == 0 && ((uintptr_t)proj & (4 * sizeof(IT) - 1)) == 0 && ((uintptr_t)out & (4 * sizeof(AT) - 1)) == 0 &&
        (!w || ((uintptr_t)w & (4 * sizeof(WT) - 1)) == 0)) {
        const int first = groups == 1 ? 0 : warp, step_g = groups == 1 ? 1 : nwarps;
        const int me = groups == 1 ? threadIdx.x : lane, n_me = groups == 1 ? blockDim.x : 32;
        for (int gi = first; gi < groups; gi += step_g) {
            float ss = 0.f;
            for (int i = me * 4; i < gw; i += n_me * 4) {
                float x[4];
                load4(row + gi * gw + i, x);
                ss += x[0] * x[0] + x[1] * x[1] + x[2] * x[2] + x[3] * x[3];
            }
            ss = groups == 1 ? block_sum(ss, scratch) : warp_sum(ss);
            const float inv = rsqrtf(ss / (float)gw + eps);
            for (int i = me * 4; i < gw; i += n_me * 4) {
                const int c = gi * gw + i;
                float x[4], z[4] = {0.f, 0.f, 0.f, 0.f}, ww[4] = {1.f, 1.f, 1.f, 1.f};
                load4(row + c, x);
                for (int s = 0; s < n_in; ++s) {
                    float p[4];
                    load4(g + (size_t)s * in_stride + c, p);
                    z[0] += p[0]; z[1] += p[1]; z[2] += p[2]; z[3] += p[3];
                }
                if (w) load4(w + c, ww);
#pragma unroll
                for (int u = 0; u < 4; ++u)
                    x[u] = x[u] * inv * ww[u] * (gate_act == 1 ? silu(z[u]) : (gate_act == 2 ? 1.f / (1.f + expf(-z[u])) : 1.f));
                store4(dst + c, x);
            }
        }
        return;
    }
    if (groups == 1) {
        float ss = 0.f;
        for (int i = threadIdx.x; i < W; i += blockDim.x) { const float x = row[i]; ss += x * x; }
        ss = block_sum(ss, scratch);
        const float inv = rsqrtf(ss / (float)W + eps);
        for (int i = threadIdx.x; i < W; i += blockDim.x) {
            float x = row[i] * inv;
            if (w) x *= to_f32(w[i]);
            const float z = load_sum(g + i, n_in, in_stride);
            x *= gate_act == 1 ? silu(z) : (gate_act == 2 ? 1.f / (1.f + expf(-z)) : 1.f);
            dst[i] = from_f32<AT>(x);
        }
        return;
    }
    for (int gi = warp; gi < groups; gi += nwarps) {
        float ss = 0.f;
        for (int i = lane; i < gw; i += 32) { const float x = row[gi * gw + i]; ss += x * x; }
        ss = warp_sum(ss);
        const float inv = rsqrtf(ss / (float)gw + eps);
        for (int i = lane; i < gw; i += 32) {
            const int c = gi * gw + i;
            float x = row[c] * inv;
            if (w) x *= to_f32(w[c]);
            const float z = load_sum(g + c, n_in, in_stride);
            x *= gate_act == 1 ? silu(z) : (gate_act == 2 ? 1.f / (1.f + expf(-z)) : 1.f);
            dst[c] = from_f32<AT>(x);
        }
    }
}
}  // namespace

// The state tile's width and the parts a column is cut in, from the sizes alone (so that a token's sums are
// always formed the same way): as many columns as keep the tile within 64 KB, at most 64; the block's 256 threads
// are dealt out over the columns, P of them a column.
static void scan_shape(int dim, int vdim, int* VT, int* P) {
    int vt = vdim < 64 ? vdim : 64;
    while (vt > 1 && (size_t)dim * vt * sizeof(float) > 64 * 1024) vt = (vt + 1) / 2;
    int p = SCAN_THREADS / vt;
    if (p > dim) p = dim;
    if (p < 1) p = 1;
    *VT = vt;
    *P = p;
}

extern "C" int rb_decay_scan(const void* in, int in_dtype, int n_in, long long in_stride, int row_stride, int q_off,
                             int k_off, int v_off, int heads, int dim, int vdim, int act_qk, int act_v, float k_scale,
                             const float* decay, float* state, const int* seq_slot, const int* cu_q, int B, float* out,
                             int ld_out, void* stream) {
    if (B <= 0) return RB_OK;
    if (heads <= 0 || dim <= 0 || vdim <= 0 || n_in < 1 || B > 65535 || heads > 65535) return RB_ERR_BAD_SIZE;
    int VT, P;
    scan_shape(dim, vdim, &VT, &P);
    if (VT > SCAN_THREADS) return RB_ERR_BAD_SIZE;
    const size_t smem = ((size_t)dim * VT + 2 * SCAN_TB * dim + SCAN_TB * VT + (size_t)SCAN_TB * P * VT) * sizeof(float);
    if (smem > 200 * 1024) return RB_ERR_BAD_SIZE;
    dim3 grid((vdim + VT - 1) / VT, heads, B);
    cudaStream_t s = (cudaStream_t)stream;
#define RB_SCAN(IT)                                                                                                      \
    do {                                                                                                                 \
        if (smem > 48 * 1024) {                                                                                          \
            cudaError_t e = cudaFuncSetAttribute(decay_scan_kernel<IT>, cudaFuncAttributeMaxDynamicSharedMemorySize,     \
                                                 (int)smem);                                                             \
            if (e != cudaSuccess) return (int)e;                                                                         \
        }                                                                                                                \
        RB_LAUNCH((decay_scan_kernel<IT>), grid, dim3(SCAN_THREADS), smem, s, (const IT*)in, n_in, (size_t)in_stride,    \
                  row_stride, q_off, k_off, v_off, heads, dim, vdim, act_qk, act_v, k_scale, decay, state, seq_slot,     \
                  cu_q, out, ld_out, VT, P);                                                                             \
    } while (0)
    if (in_dtype == RB_BF16) RB_SCAN(__nv_bfloat16);
    else if (in_dtype == RB_F32) RB_SCAN(float);
    else return RB_ERR_BAD_DTYPE;
#undef RB_SCAN
    RB_LAUNCH_CHECK();
    return RB_OK;
}

extern "C" int rb_group_norm_gate(const float* o, int ld_o, const void* proj, int proj_dtype, int n_in, long long in_stride,
                                  int row_stride, int g_off, const void* w, int w_dtype, float eps, int groups, int W,
                                  int gate_act, void* out, int out_dtype, int ld_out, const int* slot_of_token, int T,
                                  void* stream) {
    if (T <= 0) return RB_OK;
    if (groups <= 0 || W <= 0 || W % groups || n_in < 1) return RB_ERR_BAD_SIZE;
    cudaStream_t s = (cudaStream_t)stream;
    typedef __nv_bfloat16 bf;
#define RB_GNG(IT, AT, WT)                                                                                               \
    RB_LAUNCH((group_norm_gate_kernel<IT, AT, WT>), dim3(T), dim3(256), 0, s, o, ld_o, (const IT*)proj, n_in,            \
              (size_t)in_stride, row_stride, g_off, (const WT*)w, eps, groups, W, gate_act, (AT*)out, ld_out, slot_of_token)
    const bool wf = !w || w_dtype == RB_F32;
    if (proj_dtype == RB_BF16 && out_dtype == RB_BF16 && !wf) RB_GNG(bf, bf, bf);
    else if (proj_dtype == RB_BF16 && out_dtype == RB_BF16) RB_GNG(bf, bf, float);
    else if (proj_dtype == RB_F32 && out_dtype == RB_BF16 && !wf) RB_GNG(float, bf, bf);
    else if (proj_dtype == RB_F32 && out_dtype == RB_BF16) RB_GNG(float, bf, float);
    else if (proj_dtype == RB_F32 && out_dtype == RB_F32 && wf) RB_GNG(float, float, float);
    else if (proj_dtype == RB_F32 && out_dtype == RB_F32) RB_GNG(float, float, bf);
    else return RB_ERR_BAD_DTYPE;
#undef RB_GNG
    RB_LAUNCH_CHECK();
    return RB_OK;
}

// The same recurrence for prompts, by blocks of 64 tokens that run side by side (see above).  work: float32
// [blocks, heads, dim, vdim] with blocks >= the sum over the sequences of ceil(tokens / 64) (at most T / 64 + B).
// Head sizes up to 128; beyond, RB_ERR_BAD_SIZE (the caller then takes rb_decay_scan).
extern "C" int rb_decay_scan_blocks(const void* in, int in_dtype, int n_in, long long in_stride, int row_stride, int q_off,
                                    int k_off, int v_off, int heads, int dim, int vdim, int act_qk, int act_v,
                                    float k_scale, const float* decay, float* state, const int* seq_slot, const int* cu_q,
                                    int B, int max_blocks, float* work, float* out, int ld_out, void* stream) {
    if (B <= 0 || max_blocks <= 0) return RB_OK;
    if (heads <= 0 || dim <= 0 || vdim <= 0 || dim > 128 || vdim > 128 || n_in < 1 || B > 65535 || heads > 65535)
        return RB_ERR_BAD_SIZE;
    cudaStream_t s = (cudaStream_t)stream;
    const size_t smem1 = (size_t)CB * (dim + vdim) * sizeof(float);
    const size_t smem3 = ((size_t)2 * CB * dim + (size_t)CB * vdim + (size_t)CB * CB) * sizeof(float);
    const bool small = dim <= 64 && vdim <= 64;
    dim3 grid(max_blocks, heads);
#define RB_BLOCKS(IT, R)                                                                                                  \
    do {                                                                                                                  \
        cudaError_t e = cudaFuncSetAttribute(chunk_state_kernel<IT, R>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem1); \
        if (e != cudaSuccess) return (int)e;                                                                              \
        e = cudaFuncSetAttribute(chunk_out_kernel<IT, R>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem3);       \
        if (e != cudaSuccess) return (int)e;                                                                              \
        RB_LAUNCH((chunk_state_kernel<IT, R>), grid, dim3(CT), smem1, s, (const IT*)in, n_in, (size_t)in_stride, row_stride, \
                  k_off, v_off, heads, dim, vdim, act_qk, act_v, k_scale, decay, seq_slot, cu_q, B, work);                \
        if ((dim * vdim) % 4 == 0)                                                                                        \
            RB_LAUNCH((chunk_prefix_kernel<4>), dim3((dim * vdim / 4 + 255) / 256, heads, B), dim3(256), 0, s, decay, state, \
                      seq_slot, cu_q, B, heads, dim, vdim, work);                                                         \
        else                                                                                                              \
            RB_LAUNCH((chunk_prefix_kernel<1>), dim3((dim * vdim + 255) / 256, heads, B), dim3(256), 0, s, decay, state,  \
                      seq_slot, cu_q, B, heads, dim, vdim, work);                                                         \
        RB_LAUNCH((chunk_out_kernel<IT, R>), grid, dim3(CT), smem3, s, (const IT*)in, n_in, (size_t)in_stride, row_stride, \
                  q_off, k_off, v_off, heads, dim, vdim, act_qk, act_v, k_scale, decay, seq_slot, cu_q, B, work, out, ld_out); \
    } while (0)
    if (in_dtype == RB_BF16) { if (small) RB_BLOCKS(__nv_bfloat16, 4); else RB_BLOCKS(__nv_bfloat16, 8); }
    else if (in_dtype == RB_F32) { if (small) RB_BLOCKS(float, 4); else RB_BLOCKS(float, 8); }
    else return RB_ERR_BAD_DTYPE;
#undef RB_BLOCKS
    RB_LAUNCH_CHECK();
    return RB_OK;
}

// One token a sequence (a decode step): rb_decay_scan's result for sequences that bring exactly one token, with the
// state streamed through registers instead of staged in shared memory.
extern "C" int rb_decay_step(const void* in, int in_dtype, int n_in, long long in_stride, int row_stride, int q_off,
                             int k_off, int v_off, int heads, int dim, int vdim, int act_qk, int act_v, float k_scale,
                             const float* decay, float* state, const int* seq_slot, const int* cu_q, int B, float* out,
                             int ld_out, void* stream) {
    if (B <= 0) return RB_OK;
    if (heads <= 0 || dim <= 0 || vdim <= 0 || n_in < 1 || B > 65535 || heads > 65535 || dim > 4096) return RB_ERR_BAD_SIZE;
    dim3 grid((vdim + 31) / 32, heads, B);
    const size_t smem = (size_t)2 * dim * sizeof(float);
    cudaStream_t s = (cudaStream_t)stream;
    if (in_dtype == RB_BF16)
        RB_LAUNCH((decay_step_kernel<__nv_bfloat16>), grid, dim3(256), smem, s, (const __nv_bfloat16*)in, n_in, (size_t)in_stride,
                  row_stride, q_off, k_off, v_off, heads, dim, vdim, act_qk, act_v, k_scale, decay, state, seq_slot, cu_q, out, ld_out);
    else if (in_dtype == RB_F32)
        RB_LAUNCH((decay_step_kernel<float>), grid, dim3(256), smem, s, (const float*)in, n_in, (size_t)in_stride, row_stride,
                  q_off, k_off, v_off, heads, dim, vdim, act_qk, act_v, k_scale, decay, state, seq_slot, cu_q, out, ld_out);
    else
        return RB_ERR_BAD_DTYPE;
    RB_LAUNCH_CHECK();
    return RB_OK;
}
