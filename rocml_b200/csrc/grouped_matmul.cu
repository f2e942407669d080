// Many small matrix products in one launch: out_g[M_g, N] = x_g[M_g, K] . W_g[N, K]^T, one weight per group.
//
// Two ways of naming the groups:
//   * heads: group g reads columns g * x_col_stride .. + K of every row of x and writes columns
//     g * o_col_stride .. + N of the same row of out (grid.z = groups).  Used for per-head products
//     (a query folded into a latent space, a latent result unfolded into values).  `row_scale`
//     (optional, float32 [M, groups]) multiplies group g's result for row m.
//   * tiles: x holds rows sorted by group, each group's rows starting at a multiple of `tile_rows`;
//     tile_group[i] names the group of rows i * tile_rows .. (-1: an unused tile).  Used for routed
//     experts.  tile_rows is 16 (the kernels' small row tile) or a multiple of 64 (their large one).
// W is [groups][N][K], K contiguous.  Accumulation is 32-bit with k ascending, so a row's result depends on
// nothing but the row and the weight.  bfloat16 operands whose rows start on 16 bytes take the tensor cores
// (mma.sync m16n8k16, operands through padded shared-memory tiles filled by cp.async, two stages); everything
// else, and the 32-bit path always, takes the FMA kernel.
#include <cstdlib>
#include <cstring>
#include "common.cuh"
#include "mma_tiles.cuh"
#include "api.h"

using namespace rb;

namespace {
struct GP {
    const void* x; long long ldx; int x_col_stride;
    const void* w; long long w_group_stride;
    void* out; long long ldo; int o_col_stride;
    int M, N, K;
    const int* tile_group; int tile_rows;
    const float* row_scale; int row_scale_ld;
    // tensor-core kernel only: W's rows alternate in blocks of 16 between gate and up; out gets N / 2 columns,
    // act 1: silu(g) * u, act 2: min(g, limit) * sigmoid(alpha * min(g, limit)) * (clamp(u, -limit, limit) + 1)
    int act; float limit, alpha;
};

// ---- CUDA cores -------------------------------------------------------------------------------------
template <typename XT, typename WT, typename OT, int BM>
__global__ void __launch_bounds__(256)
grouped_fma_kernel(const GP p) {
    pdl_trigger();
    pdl_wait();
    constexpr int BN = 64, BK = 16, TN = 4;
    constexpr int TM = BM / 16;            // 4 (64 rows) or 1 (16 rows)
    __shared__ float xs[BK][BM + 4];
    __shared__ float ws[BK][BN + 4];
    int g = blockIdx.z;
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    int m_end = p.M;
    if (p.tile_group) {
        g = p.tile_group[m0 / p.tile_rows];
        if (g < 0) return;
        m_end = m0 + BM;
    }
    const XT* x = (const XT*)p.x + (size_t)g * p.x_col_stride;
    const WT* w = (const WT*)p.w + (size_t)g * p.w_group_stride;
    const int tid = threadIdx.x;
    const int ty = tid / 16, tx = tid % 16;
    float acc[TM][TN];
#pragma unroll
    for (int i = 0; i < TM; ++i)
#pragma unroll
        for (int j = 0; j < TN; ++j) acc[i][j] = 0.f;
    for (int k0 = 0; k0 < p.K; k0 += BK) {
        for (int idx = tid; idx < BM * BK; idx += 256) {
            const int r = idx / BK, k = idx % BK;
            const int m = m0 + r;
            xs[k][r] = (m < m_end && k0 + k < p.K) ? to_f32(x[(size_t)m * p.ldx + k0 + k]) : 0.f;
        }
        for (int idx = tid; idx < BN * BK; idx += 256) {
            const int r = idx / BK, k = idx % BK;
            const int n = n0 + r;
            ws[k][r] = (n < p.N && k0 + k < p.K) ? to_f32(w[(size_t)n * p.K + k0 + k]) : 0.f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < BK; ++kk) {
            float a[TM], b[TN];
#pragma unroll
            for (int i = 0; i < TM; ++i) a[i] = xs[kk][ty * TM + i];
#pragma unroll
            for (int j = 0; j < TN; ++j) b[j] = ws[kk][tx * TN + j];
#pragma unroll
            for (int i = 0; i < TM; ++i)
#pragma unroll
                for (int j = 0; j < TN; ++j) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
    OT* out = (OT*)p.out + (size_t)g * p.o_col_stride;
#pragma unroll
    for (int i = 0; i < TM; ++i) {
        const int m = m0 + ty * TM + i;
        if (m >= m_end) continue;
        const float sc = p.row_scale ? p.row_scale[(size_t)m * p.row_scale_ld + g] : 1.f;
#pragma unroll
        for (int j = 0; j < TN; ++j) {
            const int n = n0 + tx * TN + j;
            if (n < p.N) out[(size_t)m * p.ldo + n] = from_f32<OT>(p.row_scale ? acc[i][j] * sc : acc[i][j]);
        }
    }
}

// ---- tensor cores (bfloat16) ----------------------------------------------------------------------------
// WM x WN warps, each MT tiles of 16 rows by NT tiles of 8 columns; a k step of 32 per stage.
template <typename OT, int WM, int WN, int MT, int NT>
__global__ void __launch_bounds__(WM * WN * 32)
grouped_mma_kernel(const GP p) {
    using namespace mma_tiles;
    constexpr int BM = WM * MT * 16, BN = WN * NT * 8, BK = 32, LD = BK + 8, THREADS = WM * WN * 32;
    static_assert(NT % 2 == 0, "column tiles are loaded two at a time");
    __shared__ __align__(16) __nv_bfloat16 As[2][BM][LD];
    __shared__ __align__(16) __nv_bfloat16 Bs[2][BN][LD];
    pdl_trigger();
    pdl_wait();
    int g = blockIdx.z;
    const int m0 = blockIdx.y * BM, n0 = blockIdx.x * BN;
    int m_end = p.M;
    if (p.tile_group) {
        g = p.tile_group[m0 / p.tile_rows];
        if (g < 0) return;
        m_end = m0 + BM;
    }
    const __nv_bfloat16* x = (const __nv_bfloat16*)p.x + (size_t)g * p.x_col_stride;
    const __nv_bfloat16* w = (const __nv_bfloat16*)p.w + (size_t)g * p.w_group_stride;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int wm = warp / WN, wn = warp % WN;
    float acc[MT][NT][4];
#pragma unroll
    for (int i = 0; i < MT; ++i)
#pragma unroll
        for (int j = 0; j < NT; ++j) { acc[i][j][0] = acc[i][j][1] = acc[i][j][2] = acc[i][j][3] = 0.f; }

    auto fetch = [&](int buf, int k0) {
        for (int idx = tid; idx < BM * 4; idx += THREADS) {
            const int r = idx >> 2, c = idx & 3;
            const int m = m0 + r, k = k0 + c * 8;
            const bool ok = m < m_end && k < p.K;
            cp_async16(&As[buf][r][c * 8], x + (ok ? (size_t)m * p.ldx + k : 0), ok);
        }
        for (int idx = tid; idx < BN * 4; idx += THREADS) {
            const int r = idx >> 2, c = idx & 3;
            const int n = n0 + r, k = k0 + c * 8;
            const bool ok = n < p.N && k < p.K;
            cp_async16(&Bs[buf][r][c * 8], w + (ok ? (size_t)n * p.K + k : 0), ok);
        }
        cp_async_commit();
    };

    const int n_k = (p.K + BK - 1) / BK;
    fetch(0, 0);
    for (int kb = 0; kb < n_k; ++kb) {
        const int buf = kb & 1;
        if (kb + 1 < n_k) {
            fetch(buf ^ 1, (kb + 1) * BK);
            cp_async_wait<1>();
        } else {
            cp_async_wait<0>();
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < BK / 16; ++kk) {
            uint32_t a[MT][4];
#pragma unroll
            for (int i = 0; i < MT; ++i)
                ldmatrix_x4(smem_addr(&As[buf][(wm * MT + i) * 16 + (lane & 15)][kk * 16 + (lane >> 4) * 8]), a[i][0], a[i][1],
                            a[i][2], a[i][3]);
#pragma unroll
            for (int j = 0; j < NT; j += 2) {
                uint32_t b0, b1, b2, b3;
                ldmatrix_x4(smem_addr(&Bs[buf][(wn * NT + j) * 8 + (lane & 7) + ((lane >> 4) << 3)][kk * 16 + ((lane >> 3) & 1) * 8]),
                            b0, b1, b2, b3);
#pragma unroll
                for (int i = 0; i < MT; ++i) {
                    mma_bf16(acc[i][j], a[i], b0, b1);
                    mma_bf16(acc[i][j + 1], a[i], b2, b3);
                }
            }
        }
        __syncthreads();
    }
    OT* out = (OT*)p.out + (size_t)g * p.o_col_stride;
    if (p.act != 0) {
        // a warp's 32 columns are 16 gates and the 16 ups of the same outputs: tiles 0, 1 and tiles 2, 3
        static_assert(NT == 4, "the gated epilogue pairs tiles 0, 1 with tiles 2, 3");
        const int half = p.N >> 1;
#pragma unroll
        for (int i = 0; i < MT; ++i) {
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                const int m = m0 + (wm * MT + i) * 16 + (lane >> 2) + h * 8;
                if (m >= m_end) continue;
#pragma unroll
                for (int j = 0; j < 2; ++j) {
                    const int f = ((n0 + wn * NT * 8) >> 1) + j * 8 + (lane & 3) * 2;
#pragma unroll
                    for (int c = 0; c < 2; ++c) {
                        float gg = acc[i][j][h * 2 + c], uu = acc[i][j + 2][h * 2 + c], v;
                        if (p.act == 1) {
                            v = gg / (1.f + expf(-gg)) * uu;
                        } else {
                            gg = fminf(gg, p.limit);
                            uu = fminf(fmaxf(uu, -p.limit), p.limit);
                            v = gg / (1.f + expf(-p.alpha * gg)) * (uu + 1.f);
                        }
                        if (f + c < half) out[(size_t)m * p.ldo + f + c] = from_f32<OT>(v);
                    }
                }
            }
        }
        return;
    }
#pragma unroll
    for (int i = 0; i < MT; ++i) {
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            const int m = m0 + (wm * MT + i) * 16 + (lane >> 2) + h * 8;
            if (m >= m_end) continue;
            const float sc = p.row_scale ? p.row_scale[(size_t)m * p.row_scale_ld + g] : 1.f;
#pragma unroll
            for (int j = 0; j < NT; ++j) {
                const int n = n0 + (wn * NT + j) * 8 + (lane & 3) * 2;
                float v0 = acc[i][j][h * 2], v1 = acc[i][j][h * 2 + 1];
                if (p.row_scale) { v0 *= sc; v1 *= sc; }
                OT* dst = out + (size_t)m * p.ldo + n;
                if (sizeof(OT) == 2 && n + 1 < p.N && (((uintptr_t)dst) & 3) == 0) {
                    *reinterpret_cast<uint32_t*>(dst) = mma_tiles::pack_bf16(v0, v1);      // both columns in one store
                } else {
                    if (n < p.N) dst[0] = from_f32<OT>(v0);
                    if (n + 1 < p.N) dst[1] = from_f32<OT>(v1);
                }
            }
        }
    }
}

bool mma_enabled() {
    static const bool on = [] {
        const char* v = std::getenv("RB_GROUPED_MMA");
        return !(v && std::strcmp(v, "0") == 0);
    }();
    return on;
}

template <typename XT, typename WT, typename OT>
int launch_fma(const GP& p, int groups, int row_tiles, bool small, cudaStream_t s) {
    if (small) {
        dim3 grid((p.N + 63) / 64, row_tiles, groups);
        RB_LAUNCH((grouped_fma_kernel<XT, WT, OT, 16>), grid, dim3(256), 0, s, p);
    } else {
        dim3 grid((p.N + 63) / 64, row_tiles, groups);
        RB_LAUNCH((grouped_fma_kernel<XT, WT, OT, 64>), grid, dim3(256), 0, s, p);
    }
    RB_LAUNCH_CHECK();
    return RB_OK;
}

template <typename OT>
int launch_mma(const GP& p, int groups, int row_tiles, bool small, cudaStream_t s) {
    if (!small && !p.tile_group && p.M >= 512 && p.N >= 128) {
        // many rows, head by head: tiles of 128 x 128, eight warps of 64 x 32
        dim3 grid((p.N + 127) / 128, (p.M + 127) / 128, groups);
        RB_LAUNCH((grouped_mma_kernel<OT, 2, 4, 4, 4>), grid, dim3(256), 0, s, p);
        RB_LAUNCH_CHECK();
        return RB_OK;
    }
    if (small) {
        dim3 grid((p.N + 127) / 128, row_tiles, groups);
        RB_LAUNCH((grouped_mma_kernel<OT, 1, 4, 1, 4>), grid, dim3(128), 0, s, p);
    } else {
        dim3 grid((p.N + 63) / 64, row_tiles, groups);
        RB_LAUNCH((grouped_mma_kernel<OT, 2, 2, 2, 4>), grid, dim3(128), 0, s, p);
    }
    RB_LAUNCH_CHECK();
    return RB_OK;
}
}  // namespace

// act != 0 (bfloat16 operands on the tensor cores only, N a multiple of 32, W's gate and up rows interleaved in
// blocks of 16): out has N / 2 columns, the gated activation of the product; RB_ERR_BAD_SIZE when the operands take
// the FMA kernel, which has no such epilogue.
// groups > 0, tile_group absent: the heads form (M rows).  tile_group given: the tiles form; M is then the
// number of rows the buffers hold (n_tiles * tile_rows) and tile_rows is 16 or a multiple of 64.
extern "C" int rb_grouped_matmul(const void* x, int x_dtype, long long ldx, int x_col_stride, const void* w, int w_dtype,
                                 long long w_group_stride, void* out, int out_dtype, long long ldo, int o_col_stride,
                                 int M, int N, int K, int groups, const int* tile_group, int tile_rows,
                                 const float* row_scale, int row_scale_ld, int act, float limit, float alpha,
                                 void* stream) {
    if (M <= 0 || N <= 0 || groups <= 0) return RB_OK;
    if (K <= 0) return RB_ERR_BAD_SIZE;
    if (tile_group && tile_rows != 16 && (tile_rows <= 0 || tile_rows % 64)) return RB_ERR_BAD_SIZE;
    cudaStream_t s = (cudaStream_t)stream;
    GP p;
    p.x = x; p.ldx = ldx; p.x_col_stride = x_col_stride;
    p.w = w; p.w_group_stride = w_group_stride;
    p.out = out; p.ldo = ldo; p.o_col_stride = o_col_stride;
    p.M = M; p.N = N; p.K = K;
    p.tile_group = tile_group; p.tile_rows = tile_rows;
    p.row_scale = row_scale; p.row_scale_ld = row_scale_ld;
    p.act = act; p.limit = limit; p.alpha = alpha;
    const bool small = tile_group ? tile_rows == 16 : M <= 16;
    const int bm = small ? 16 : 64;
    const long long row_tiles = tile_group ? M / bm : (M + bm - 1) / bm;
    const int z = tile_group ? 1 : groups;
    if (row_tiles > 65535 || z > 65535) return RB_ERR_BAD_SIZE;
    typedef __nv_bfloat16 bf;
    if (x_dtype == RB_BF16 && w_dtype == RB_BF16 && mma_enabled() && K % 8 == 0 && ldx % 8 == 0 && x_col_stride % 8 == 0 &&
        w_group_stride % 8 == 0 && (((uintptr_t)x | (uintptr_t)w) & 15) == 0) {
        if (act != 0 && (N % 32 || act > 2 || row_scale)) return RB_ERR_BAD_SIZE;
        if (out_dtype == RB_BF16) return launch_mma<bf>(p, z, (int)row_tiles, small, s);
        if (out_dtype == RB_F32) return launch_mma<float>(p, z, (int)row_tiles, small, s);
        return RB_ERR_BAD_DTYPE;
    }
    if (act != 0) return RB_ERR_BAD_SIZE;       // only the tensor-core kernel has the gated epilogue
#define RB_GF(XT, WT, OT) return launch_fma<XT, WT, OT>(p, z, (int)row_tiles, small, s)
    if (x_dtype == RB_F32 && w_dtype == RB_F32 && out_dtype == RB_F32) RB_GF(float, float, float);
    if (x_dtype == RB_BF16 && w_dtype == RB_BF16 && out_dtype == RB_BF16) RB_GF(bf, bf, bf);
    if (x_dtype == RB_BF16 && w_dtype == RB_BF16 && out_dtype == RB_F32) RB_GF(bf, bf, float);
    if (x_dtype == RB_F32 && w_dtype == RB_BF16 && out_dtype == RB_F32) RB_GF(float, bf, float);
#undef RB_GF
    return RB_ERR_BAD_DTYPE;
}
