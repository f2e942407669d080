// Routing of tokens to experts: scores and choice, the plan of rows, the gather and the weighted sum.
//
//   route    one warp a token: s_e = sigmoid(z_e) (z: 32-bit router logits); the `top` experts with the
//            largest s_e + bias_e are chosen (ties: the lower number), their weights are s_e (without the
//            bias, not renormalised).  Each choice also takes the next free place among its expert's rows
//            (an atomic counter: the order of an expert's rows is arbitrary, and no result depends on it,
//            because every row is computed by itself).  Padding tokens (slot -1) choose nothing.
//            With `n_groups` > 1 the experts form that many equal groups of neighbours; a group's score is the
//            sum of its two largest s_e + bias_e (of its only one, in groups of one), and only experts of the
//            `keep_groups` best groups (ties: the lower number) can be chosen.  With `renormalize` the weights
//            are divided by their sum + norm_eps.
//   plan     one block: every expert's rows start at a multiple of `tile_rows`; tile i of the row buffer
//            belongs to expert tile_group[i] (-1: unused).
//   gather   a token's normalised row is copied to each of its `top` places; row_of[t, j] names the place.
//   combine  out[t] = sum_j weight[t, j] * y[row_of[t, j]] in 32-bit, j ascending; optionally plus
//            sigmoid(extra_gate[t]) * (sum of the partial sums extra[s][t]): an expert that every token uses.
#include "common.cuh"
#include "api.h"

using namespace rb;

namespace {
constexpr int MAX_EPL = 16;   // experts per lane: up to 512 experts

// ---- router logits: z[t, e] = sum_k x[t, k] * w[e, k], 32-bit FMA, w float32 ---------------------------------
// A block takes TT tokens (their rows staged in shared memory as float32) and 8 * EW experts, a warp EW of them:
// a lane takes its slice of k of the block's tokens from shared memory once and multiplies it with the same slice
// of each of its experts' rows, which it streams with 16-byte loads; the lanes' sums meet in a shuffle tree.  How
// k is dealt out depends on K only, so a token's logits depend on nothing else in the batch.  EW is 1 for a
// handful of tokens (more blocks stream the router's rows) and 4 beyond (a quarter of the shared-memory reads).
constexpr int RT_WARPS = 8;

template <typename XT, int TT, int EW>
__global__ void __launch_bounds__(RT_WARPS * 32)
router_logits_kernel(const XT* __restrict__ x, long long ldx, const float* __restrict__ w, float* __restrict__ z, int ldz,
                     int T, int E, int K) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ __align__(16) float xs[];      // [TT][K]
    const int t0 = blockIdx.x * TT;
    if (sizeof(XT) == 2 && (K & 7) == 0 && (ldx & 7) == 0 && ((uintptr_t)x & 15) == 0) {
        const int K8 = K >> 3;
        for (int idx = threadIdx.x; idx < TT * K8; idx += blockDim.x) {
            const int r = idx / K8, c = idx - r * K8;
            uint4 raw = make_uint4(0u, 0u, 0u, 0u);
            if (t0 + r < T) raw = *reinterpret_cast<const uint4*>(reinterpret_cast<const uint16_t*>(x) + (size_t)(t0 + r) * ldx + c * 8);
            const uint32_t ws[4] = {raw.x, raw.y, raw.z, raw.w};
            float* d = xs + (size_t)r * K + c * 8;
#pragma unroll
            for (int i = 0; i < 4; ++i) {
                d[2 * i] = __uint_as_float(ws[i] << 16);
                d[2 * i + 1] = __uint_as_float(ws[i] & 0xFFFF0000u);
            }
        }
    } else {
        for (int idx = threadIdx.x; idx < TT * K; idx += blockDim.x) {
            const int r = idx / K, k = idx - r * K;
            xs[idx] = t0 + r < T ? to_f32(x[(size_t)(t0 + r) * ldx + k]) : 0.f;
        }
    }
    __syncthreads();
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const int e0 = (blockIdx.y * RT_WARPS + warp) * EW;
    if (e0 >= E) return;
    float acc[EW][TT];
#pragma unroll
    for (int j = 0; j < EW; ++j)
#pragma unroll
        for (int r = 0; r < TT; ++r) acc[j][r] = 0.f;
    if ((K & 3) == 0 && ((uintptr_t)w & 15) == 0) {
        const int K4 = K >> 2;
        for (int k4 = lane; k4 < K4; k4 += 32) {
            float4 wv[EW];
#pragma unroll
            for (int j = 0; j < EW; ++j)
                wv[j] = e0 + j < E ? reinterpret_cast<const float4*>(w + (size_t)(e0 + j) * K)[k4] : make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
            for (int r = 0; r < TT; ++r) {
                const float4 xv = *reinterpret_cast<const float4*>(xs + (size_t)r * K + (size_t)k4 * 4);
#pragma unroll
                for (int j = 0; j < EW; ++j) {
                    acc[j][r] = fmaf(wv[j].x, xv.x, acc[j][r]);
                    acc[j][r] = fmaf(wv[j].y, xv.y, acc[j][r]);
                    acc[j][r] = fmaf(wv[j].z, xv.z, acc[j][r]);
                    acc[j][r] = fmaf(wv[j].w, xv.w, acc[j][r]);
                }
            }
        }
    } else {
        for (int k = lane; k < K; k += 32) {
#pragma unroll
            for (int j = 0; j < EW; ++j) {
                const float wv = e0 + j < E ? w[(size_t)(e0 + j) * K + k] : 0.f;
#pragma unroll
                for (int r = 0; r < TT; ++r) acc[j][r] = fmaf(wv, xs[(size_t)r * K + k], acc[j][r]);
            }
        }
    }
#pragma unroll
    for (int j = 0; j < EW; ++j)
#pragma unroll
        for (int r = 0; r < TT; ++r) {
            const float v = warp_sum(acc[j][r]);
            if (lane == 0 && t0 + r < T && e0 + j < E) z[(size_t)(t0 + r) * ldz + e0 + j] = v;
        }
}

template <typename XT, int TT>
int launch_router(const void* x, long long ldx, const float* w, float* z, int ldz, int T, int E, int K, cudaStream_t s) {
    const size_t smem = (size_t)TT * K * sizeof(float);
    const bool few = T <= 16;
    auto k = few ? router_logits_kernel<XT, TT, 1> : router_logits_kernel<XT, TT, 4>;
    if (smem > 48 * 1024) {
        cudaError_t e = cudaFuncSetAttribute(k, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
        if (e != cudaSuccess) return (int)e;
    }
    const int per_block = RT_WARPS * (few ? 1 : 4);
    dim3 grid((T + TT - 1) / TT, (E + per_block - 1) / per_block);
    if (grid.y > 65535) return RB_ERR_BAD_SIZE;
    RB_LAUNCH((k), grid, dim3(RT_WARPS * 32), smem, s, (const XT*)x, ldx, w, z, ldz, T, E, K);
    RB_LAUNCH_CHECK();
    return RB_OK;
}

template <typename BT>
__global__ void __launch_bounds__(128)
moe_route_kernel(const float* __restrict__ z, int ldz, const BT* __restrict__ bias, const int* __restrict__ slot_of_token,
                 int T, int E, int top, int* __restrict__ ids, float* __restrict__ weights, int* __restrict__ place,
                 int* __restrict__ counts, int n_groups, int keep_groups, int renormalize, float norm_eps) {
    pdl_trigger();
    pdl_wait();
    extern __shared__ float route_s[];           // [warps][E + n_groups] when groups are cut, else unused
    const int t = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
    const int lane = threadIdx.x & 31;
    if (t >= T) return;
    if (slot_of_token[t] < 0) {
        for (int j = lane; j < top; j += 32) { ids[(size_t)t * top + j] = -1; weights[(size_t)t * top + j] = 0.f; place[(size_t)t * top + j] = 0; }
        return;
    }
    float s[MAX_EPL], c[MAX_EPL];
#pragma unroll
    for (int i = 0; i < MAX_EPL; ++i) {
        const int e = lane + i * 32;
        if (e < E) {
            s[i] = 1.f / (1.f + expf(-z[(size_t)t * ldz + e]));
            c[i] = s[i] + (bias ? to_f32(bias[e]) : 0.f);
        } else {
            s[i] = 0.f;
            c[i] = -INFINITY;
        }
    }
    if (n_groups > 1 && keep_groups < n_groups) {
        // the groups' cut: scores to shared memory, a lane scores whole groups, the best groups are marked
        float* cs = route_s + (size_t)(threadIdx.x >> 5) * (E + n_groups);
        float* gs = cs + E;
        const int per = E / n_groups;
#pragma unroll
        for (int i = 0; i < MAX_EPL; ++i)
            if (lane + i * 32 < E) cs[lane + i * 32] = c[i];
        __syncwarp();
        for (int g = lane; g < n_groups; g += 32) {
            float a = -INFINITY, b = -INFINITY;       // the two largest
            for (int e = g * per; e < (g + 1) * per; ++e) {
                const float v = cs[e];
                if (v > a) { b = a; a = v; } else if (v > b) b = v;
            }
            gs[g] = per > 1 ? a + b : a;
        }
        __syncwarp();
        for (int j = 0; j < keep_groups; ++j) {
            float best = -INFINITY;
            int best_g = 0x7fffffff;
            for (int g = lane; g < n_groups; g += 32)
                if (gs[g] > best) { best = gs[g]; best_g = g; }
#pragma unroll
            for (int o = 16; o > 0; o >>= 1) {
                const float ob = __shfl_xor_sync(0xffffffffu, best, o);
                const int og = __shfl_xor_sync(0xffffffffu, best_g, o);
                if (ob > best || (ob == best && og < best_g)) { best = ob; best_g = og; }
            }
            __syncwarp();
            if (lane == 0 && best_g < n_groups) gs[best_g] = -INFINITY;     // kept: marked by -inf, not NaN
            __syncwarp();
        }
#pragma unroll
        for (int i = 0; i < MAX_EPL; ++i) {
            const int e = lane + i * 32;
            if (e < E && gs[e / per] != -INFINITY) c[i] = -INFINITY;       // its group was not kept
        }
    }
    float picked_sum = 0.f;
    for (int j = 0; j < top; ++j) {
        float best = -INFINITY, best_s = 0.f;
        int best_e = 0x7fffffff;
#pragma unroll
        for (int i = 0; i < MAX_EPL; ++i) {
            const int e = lane + i * 32;
            if (e < E && (c[i] > best)) { best = c[i]; best_e = e; best_s = s[i]; }   // ascending e: the first of equals stays
        }
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const int oe = __shfl_xor_sync(0xffffffffu, best_e, o);
            const float os = __shfl_xor_sync(0xffffffffu, best_s, o);
            if (ob > best || (ob == best && oe < best_e)) { best = ob; best_e = oe; best_s = os; }
        }
#pragma unroll
        for (int i = 0; i < MAX_EPL; ++i)
            if (lane + i * 32 == best_e) c[i] = -INFINITY;
        if (best_e >= E) best_e = E - 1;      // scores that compare with nothing (NaN): stay inside the tables
        picked_sum += best_s;
        if (lane == 0) {
            ids[(size_t)t * top + j] = best_e;
            weights[(size_t)t * top + j] = best_s;
            place[(size_t)t * top + j] = atomicAdd(&counts[best_e], 1);
        }
    }
    if (renormalize && lane == 0) {
        const float d = picked_sum + norm_eps;
        for (int j = 0; j < top; ++j) weights[(size_t)t * top + j] /= d;
    }
}

__global__ void __launch_bounds__(256)
moe_plan_kernel(const int* __restrict__ counts, int E, int tile_rows, int max_tiles, int* __restrict__ starts,
                int* __restrict__ tile_group) {
    pdl_trigger();
    pdl_wait();
    for (int i = threadIdx.x; i < max_tiles; i += blockDim.x) tile_group[i] = -1;
    __syncthreads();
    if (threadIdx.x == 0) {
        int tile = 0;
        for (int e = 0; e < E; ++e) {
            starts[e] = tile * tile_rows;
            const int n = (counts[e] + tile_rows - 1) / tile_rows;
            for (int i = 0; i < n && tile + i < max_tiles; ++i) tile_group[tile + i] = e;
            tile += n;
        }
        starts[E] = tile * tile_rows;
    }
}

template <typename AT>
__global__ void __launch_bounds__(128)
moe_gather_kernel(const AT* __restrict__ x, int H, const int* __restrict__ ids, const int* __restrict__ place,
                  const int* __restrict__ starts, int top, AT* __restrict__ rows, int* __restrict__ row_of) {
    pdl_trigger();
    pdl_wait();
    const int tj = blockIdx.x;
    const int e = ids[tj];
    if (e < 0) {
        if (threadIdx.x == 0) row_of[tj] = -1;
        return;
    }
    const int r = starts[e] + place[tj];
    if (threadIdx.x == 0) row_of[tj] = r;
    const AT* src = x + (size_t)(tj / top) * H;
    AT* dst = rows + (size_t)r * H;
    if ((H * sizeof(AT)) % 16 == 0 && (((uintptr_t)x | (uintptr_t)rows) & 15) == 0) {
        const int n16 = (int)(H * sizeof(AT) / 16);
        for (int i = threadIdx.x; i < n16; i += blockDim.x)
            reinterpret_cast<uint4*>(dst)[i] = reinterpret_cast<const uint4*>(src)[i];
    } else {
        for (int i = threadIdx.x; i < H; i += blockDim.x) dst[i] = src[i];
    }
}

__global__ void __launch_bounds__(256)
moe_combine_kernel(const float* __restrict__ y, long long ldy, const int* __restrict__ row_of, const float* __restrict__ weights,
                   int top, float* __restrict__ out, int H, const float* __restrict__ extra, int n_extra,
                   long long extra_stride, const float* __restrict__ extra_gate, int extra_gate_ld) {
    pdl_trigger();
    pdl_wait();
    const int t = blockIdx.x;
    const float eg = extra ? (extra_gate ? 1.f / (1.f + expf(-extra_gate[(size_t)t * extra_gate_ld])) : 1.f) : 0.f;
    for (int i = threadIdx.x; i < H; i += blockDim.x) {
        float v = 0.f;
        for (int j = 0; j < top; ++j) {
            const int r = row_of[(size_t)t * top + j];
            if (r >= 0) v = fmaf(weights[(size_t)t * top + j], y[(size_t)r * ldy + i], v);
        }
        if (extra) {
            float x = 0.f;
            for (int s = 0; s < n_extra; ++s) x += extra[(size_t)s * extra_stride + (size_t)t * H + i];
            v = fmaf(eg, x, v);
        }
        out[(size_t)t * H + i] = v;
    }
}
}  // namespace

extern "C" int rb_router_logits(const void* x, int x_dtype, long long ldx, const float* w, float* z, int ldz, int T, int E,
                                int K, void* stream) {
    if (T <= 0 || E <= 0) return RB_OK;
    if (K <= 0) return RB_ERR_BAD_SIZE;
    cudaStream_t s = (cudaStream_t)stream;
    // tokens a block: as many as fit 96 KB of shared memory, at most 8
    const int fit = (int)((96 * 1024) / ((size_t)K * sizeof(float)));
    if (fit < 1) return RB_ERR_BAD_SIZE;
    const int tt = fit >= 8 ? 8 : (fit >= 4 ? 4 : (fit >= 2 ? 2 : 1));
#define RB_RL(XT)                                                                         \
    switch (tt) {                                                                         \
        case 8: return launch_router<XT, 8>(x, ldx, w, z, ldz, T, E, K, s);               \
        case 4: return launch_router<XT, 4>(x, ldx, w, z, ldz, T, E, K, s);               \
        case 2: return launch_router<XT, 2>(x, ldx, w, z, ldz, T, E, K, s);               \
        default: return launch_router<XT, 1>(x, ldx, w, z, ldz, T, E, K, s);              \
    }
    if (x_dtype == RB_BF16) { RB_RL(__nv_bfloat16) }
    if (x_dtype == RB_F32) { RB_RL(float) }
#undef RB_RL
    return RB_ERR_BAD_DTYPE;
}

extern "C" int rb_moe_route(const float* z, int ldz, const void* bias, int bias_dtype, const int* slot_of_token, int T,
                            int E, int top, int* ids, float* weights, int* place, int* counts, int n_groups,
                            int keep_groups, int renormalize, float norm_eps, void* stream) {
    if (T <= 0) return RB_OK;
    if (E <= 0 || E > 32 * MAX_EPL || top <= 0 || top > E) return RB_ERR_BAD_SIZE;
    if (n_groups < 1) n_groups = 1;
    if (keep_groups < 1 || keep_groups > n_groups) keep_groups = n_groups;
    if (E % n_groups || (long long)keep_groups * (E / n_groups) < top) return RB_ERR_BAD_SIZE;
    cudaStream_t s = (cudaStream_t)stream;
    const int warps = 4;
    dim3 grid((T + warps - 1) / warps);
    const size_t smem = (n_groups > 1 && keep_groups < n_groups) ? (size_t)warps * (E + n_groups) * sizeof(float) : 0;
    if (!bias || bias_dtype == RB_F32)
        RB_LAUNCH((moe_route_kernel<float>), grid, dim3(warps * 32), smem, s, z, ldz, (const float*)bias, slot_of_token, T, E, top,
                  ids, weights, place, counts, n_groups, keep_groups, renormalize, norm_eps);
    else if (bias_dtype == RB_BF16)
        RB_LAUNCH((moe_route_kernel<__nv_bfloat16>), grid, dim3(warps * 32), smem, s, z, ldz, (const __nv_bfloat16*)bias,
                  slot_of_token, T, E, top, ids, weights, place, counts, n_groups, keep_groups, renormalize, norm_eps);
    else
        return RB_ERR_BAD_DTYPE;
    RB_LAUNCH_CHECK();
    return RB_OK;
}

extern "C" int rb_moe_plan(const int* counts, int E, int tile_rows, int max_tiles, int* starts, int* tile_group,
                           void* stream) {
    if (E <= 0 || tile_rows <= 0 || max_tiles <= 0) return RB_ERR_BAD_SIZE;
    RB_LAUNCH((moe_plan_kernel), dim3(1), dim3(256), 0, (cudaStream_t)stream, counts, E, tile_rows, max_tiles, starts, tile_group);
    RB_LAUNCH_CHECK();
    return RB_OK;
}

extern "C" int rb_moe_gather(const void* x, int dtype, int H, const int* ids, const int* place, const int* starts, int T,
                             int top, void* rows, int* row_of, void* stream) {
    if (T <= 0) return RB_OK;
    cudaStream_t s = (cudaStream_t)stream;
    if (dtype == RB_BF16)
        RB_LAUNCH((moe_gather_kernel<__nv_bfloat16>), dim3(T * top), dim3(128), 0, s, (const __nv_bfloat16*)x, H, ids, place,
                  starts, top, (__nv_bfloat16*)rows, row_of);
    else if (dtype == RB_F32)
        RB_LAUNCH((moe_gather_kernel<float>), dim3(T * top), dim3(128), 0, s, (const float*)x, H, ids, place, starts, top,
                  (float*)rows, row_of);
    else
        return RB_ERR_BAD_DTYPE;
    RB_LAUNCH_CHECK();
    return RB_OK;
}

extern "C" int rb_moe_combine(const float* y, long long ldy, const int* row_of, const float* weights, int T, int top,
                              float* out, int H, const float* extra, int n_extra, long long extra_stride,
                              const float* extra_gate, int extra_gate_ld, void* stream) {
    if (T <= 0) return RB_OK;
    RB_LAUNCH((moe_combine_kernel), dim3(T), dim3(256), 0, (cudaStream_t)stream, y, ldy, row_of, weights, top, out, H,
              extra, n_extra, extra_stride, extra_gate, extra_gate_ld);
    RB_LAUNCH_CHECK();
    return RB_OK;
}
