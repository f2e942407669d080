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
