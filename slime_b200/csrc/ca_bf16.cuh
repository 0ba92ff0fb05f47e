// bf16 path of the CA step: bf16 storage of state, weights and intermediates, fp32 accumulation and stencil
// math, projections on the 5th-generation tensor cores (tcgen05.mma, accumulators in TMEM, weight tiles
// fetched by TMA).  Same two-kernel split as the fp32 path (ca_f32.cuh):
//
//   k1_bf16  per 8x16-cell tile (128 cells = UMMA M): state halo tile -> per head the 3x3-convolved input as a
//            swizzled K-major A operand; U = conv_h(X) Wp_h (N=64) and I|V = X [Wi_h|Wv_h] (N=128) into 192
//            TMEM columns; epilogue: growth bell, E = exp(G*I), write E and V (bf16, per-head planar).
//   k2_bf16  per tile and head: E (2-cell halo) and V (1-cell halo) by cp.async; separable box sums marching
//            down columns: R = V / box3(E), V' = E * box3(R); V' is the A operand of Y += V'_h Wo_h (N=64)
//            accumulated in TMEM over the 8 heads; epilogue: X+ = scale*X + dt*Y (bf16), per-tile channel sums.
//
// Shared-memory operand tiles are [rows][128 B] with the 128-byte swizzle: the 16-byte chunk q of row m
// lives at m*128 + ((q ^ (m & 7)) << 4), tile bases 1024-byte aligned.
#pragma once
#include <cuda.h>

#include "common.cuh"
#include "ptx.cuh"

namespace slime {

constexpr int TBH = 8, TBW = 16;      // tile: 8 rows x 16 columns = 128 cells
constexpr int K1B_THREADS = 256;
constexpr int K2B_THREADS = 288;
constexpr float LOG2E = 1.4426950408889634f;

struct Bf16Plan {
    int tiles_x = 1, k1_tiles = 1, k2_tiles = 1;
    CUtensorMap map_w1;   // [sets*8*192][64] bf16, box 64 x 192, 128B swizzle
    CUtensorMap map_wo;   // [sets*8*64][64]  bf16, box 64 x 64,  128B swizzle
};

// ---- shared-memory maps (byte offsets from a 1024-aligned base) -------------------------------------------
namespace k1b {
constexpr int A_X = 0, A_CONV = 16384, W0 = 32768, W_STAGE = 24576, XH = W0 + 2 * W_STAGE;   // 81920
constexpr int XH_BYTES = 10 * 18 * 128;                                                          // 23040
constexpr int SCALE = XH + XH_BYTES, PRM_S = SCALE + 256, BARS = PRM_S + NH * PRM * 4, TMEM_PTR = BARS + 32;
constexpr int BYTES = TMEM_PTR + 16;
constexpr int SMEM = BYTES + 1024;    // slack for manual 1024-byte alignment
constexpr uint32_t TMEM_COLS = 256;
}  // namespace k1b
namespace k2b {
constexpr int A_VP = 0, WO0 = 16384, WO_STAGE = 8192, ES = WO0 + 2 * WO_STAGE;   // 32768
constexpr int ES_BYTES = 12 * 20 * 128, VS = ES + ES_BYTES, VS_BYTES = 10 * 18 * 128;
constexpr int SCALE = VS + VS_BYTES, BARS = SCALE + 256, TMEM_PTR = BARS + 32;
constexpr int BYTES = TMEM_PTR + 16;
constexpr int SMEM = BYTES + 1024;
constexpr uint32_t TMEM_COLS = 64;
static_assert(ES_BYTES + VS_BYTES >= 128 * 64 * 4, "the channel-sum scratch aliases the E and V tiles");
}  // namespace k2b

__device__ __forceinline__ void unpack8(const uint4& v, float (&f)[8]) {
    f[0] = bf16_lo(v.x); f[1] = bf16_hi(v.x); f[2] = bf16_lo(v.y); f[3] = bf16_hi(v.y);
    f[4] = bf16_lo(v.z); f[5] = bf16_hi(v.z); f[6] = bf16_lo(v.w); f[7] = bf16_hi(v.w);
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
    return make_uint4(pack_bf16(f[0], f[1]), pack_bf16(f[2], f[3]), pack_bf16(f[4], f[5]), pack_bf16(f[6], f[7]));
}
__device__ __forceinline__ uint8_t* align1024(uint8_t* p) {
    return reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(p) + 1023) & ~uintptr_t(1023));
}
__device__ __forceinline__ uint32_t swz(int m, int q) { return (uint32_t)(m * 128 + ((q ^ (m & 7)) << 4)); }

// =============================================================================================================
__global__ void __launch_bounds__(K1B_THREADS, 2)
k1_bf16(const __grid_constant__ CUtensorMap map_w1, const __nv_bfloat16* __restrict__ X,
        const float* __restrict__ scale, const float* __restrict__ prm, __nv_bfloat16* __restrict__ E,
        __nv_bfloat16* __restrict__ V, int* __restrict__ status, Geom g) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* sm = align1024(smem_raw);
    uint8_t* a_x = sm + k1b::A_X;
    uint8_t* a_conv = sm + k1b::A_CONV;
    uint8_t* xh = sm + k1b::XH;
    float* scale_s = reinterpret_cast<float*>(sm + k1b::SCALE);
    float* prm_s = reinterpret_cast<float*>(sm + k1b::PRM_S);
    uint64_t* full = reinterpret_cast<uint64_t*>(sm + k1b::BARS);      // [2] weight stages
    uint64_t* mma_bar = full + 2;
    uint32_t* tmem_ptr = reinterpret_cast<uint32_t*>(sm + k1b::TMEM_PTR);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int b = blockIdx.y;
    const int tx0 = (blockIdx.x % g.tiles_x) * TBW;
    const int ty0 = (blockIdx.x / g.tiles_x) * TBH - g.he;
    const int set = b / g.per_set;
    const size_t xplane = (size_t)g.state_rows() * g.W * NC;
    const size_t eplane = (size_t)g.ev_rows() * g.W * HD;

    if (tid == 0) {
        ptx::mbar_init(&full[0], 1);
        ptx::mbar_init(&full[1], 1);
        ptx::mbar_init(mma_bar, 1);
        ptx::fence_barrier_init();
        ptx::prefetch_tmap(&map_w1);
    }
    if (warp == 0) ptx::tmem_alloc(tmem_ptr, k1b::TMEM_COLS);
    if (tid < NC) scale_s[tid] = scale[b * NC + tid];
    if (tid < NH * PRM) prm_s[tid] = prm[(size_t)set * NH * PRM + tid];
    ptx::tc_fence_before();
    __syncthreads();
    ptx::tc_fence_after();
    const uint32_t tmem = *tmem_ptr;

    if (tid == 0) {
        for (int s = 0; s < 2; ++s) {
            ptx::mbar_expect_tx(&full[s], k1b::W_STAGE);
            ptx::tma_load_2d(sm + k1b::W0 + s * k1b::W_STAGE, &map_w1, 0, (set * NH + s) * 192, &full[s]);
        }
    }

    // state halo tile (10 x 18 cells), pending renormalisation scale applied, kept as bf16
    for (int i = tid; i < 180 * 8; i += K1B_THREADS) {
        const int q = i & 7, cell = i >> 3;
        const int hy = cell / 18, hx = cell % 18;
        const int r = ty0 + hy - 1, x = g.wrap_x(tx0 + hx - 1);
        const uint4 raw = *reinterpret_cast<const uint4*>(X + (size_t)b * xplane + ((size_t)g.xrow(r) * g.W + x) * NC + q * 8);
        float f[8];
        unpack8(raw, f);
#pragma unroll
        for (int k = 0; k < 8; ++k) f[k] *= scale_s[q * 8 + k];
        const uint4 v = pack8(f);
        *reinterpret_cast<uint4*>(xh + cell * 128 + q * 16) = v;
        if (hy >= 1 && hy <= TBH && hx >= 1 && hx <= TBW)
            *reinterpret_cast<uint4*>(a_x + swz((hy - 1) * TBW + hx - 1, q)) = v;
    }
    ptx::fence_proxy_async();
    __syncthreads();

    const uint32_t idesc_u = ptx::umma_idesc_bf16(128, 64);
    const uint32_t idesc_iv = ptx::umma_idesc_bf16(128, 128);
    const int quad = warp & 3, half = warp >> 2;
    const int m_ep = quad * 32 + lane;                     // TMEM lane = cell of the tile this thread finishes
    const int r_ep = ty0 + (m_ep >> 4), x_ep = tx0 + (m_ep & 15);
    const bool valid_ep = r_ep < g.H + g.he && x_ep < g.W;
    const uint32_t t_lane = tmem + ((uint32_t)(quad * 32) << 16);

    for (int h = 0; h < NH; ++h) {
        // ---- 3x3 stencil of head h on the state tile -> A operand ------------------------------------------
        float kt[9];
#pragma unroll
        for (int t = 0; t < 9; ++t) kt[t] = prm_s[h * PRM + t];
#pragma unroll 1
        for (int pass = 0; pass < 4; ++pass) {
            const int m = pass * 32 + (tid >> 3), q = tid & 7;
            const int cy = m >> 4, cx = m & 15;
            float acc[8];
#pragma unroll
            for (int k = 0; k < 8; ++k) acc[k] = 0.f;
#pragma unroll
            for (int t = 0; t < 9; ++t) {
                const uint4 raw = *reinterpret_cast<const uint4*>(xh + ((cy + t / 3) * 18 + cx + t % 3) * 128 + q * 16);
                float f[8];
                unpack8(raw, f);
#pragma unroll
                for (int k = 0; k < 8; ++k) acc[k] = fmaf(kt[t], f[k], acc[k]);
            }
            *reinterpret_cast<uint4*>(a_conv + swz(m, q)) = pack8(acc);
        }
        ptx::fence_proxy_async();
        __syncthreads();

        // ---- projections: U | I | V into TMEM columns [0,64) | [64,128) | [128,192) -------------------------
        if (tid == 0) {
            ptx::mbar_wait(&full[h & 1], (h >> 1) & 1, status, 101);
            ptx::tc_fence_after();
            const uint32_t wb = ptx::smem_u32(sm + k1b::W0 + (h & 1) * k1b::W_STAGE);
            const uint64_t da = ptx::umma_desc_sw128(ptx::smem_u32(a_conv));
            const uint64_t dx = ptx::umma_desc_sw128(ptx::smem_u32(a_x));
            const uint64_t dwp = ptx::umma_desc_sw128(wb);
            const uint64_t dwiv = ptx::umma_desc_sw128(wb + 64 * 128);
#pragma unroll
            for (int k = 0; k < 4; ++k) ptx::umma_bf16(tmem, da + 2 * k, dwp + 2 * k, idesc_u, k > 0);
#pragma unroll
            for (int k = 0; k < 4; ++k) ptx::umma_bf16(tmem + 64, dx + 2 * k, dwiv + 2 * k, idesc_iv, k > 0);
            ptx::umma_commit(mma_bar);
        }
        ptx::mbar_wait(mma_bar, h & 1, status, 102);
        ptx::tc_fence_after();
        if (tid == 0 && h + 2 < NH) {       // the stage just consumed is free: fetch the weights of head h+2
            ptx::mbar_expect_tx(&full[h & 1], k1b::W_STAGE);
            ptx::tma_load_2d(sm + k1b::W0 + (h & 1) * k1b::W_STAGE, &map_w1, 0, (set * NH + h + 2) * 192, &full[h & 1]);
        }

        // ---- epilogue: growth bell, activation, E = exp(A); E and V to global ---------------------------------
        const float mu = prm_s[h * PRM + 9], nisl2 = prm_s[h * PRM + 10] * LOG2E;
        const size_t obase = ((size_t)b * NH + h) * eplane + ((size_t)g.erow(r_ep) * g.W + (valid_ep ? x_ep : 0)) * HD;
#pragma unroll
        for (int sub = 0; sub < 2; ++sub) {
            const int c0 = half * 32 + sub * 16;
            uint32_t ru[16], ri[16], rv[16];
            ptx::tmem_ld16(t_lane + c0, ru);
            ptx::tmem_ld16(t_lane + 64 + c0, ri);
            ptx::tmem_ld16(t_lane + 128 + c0, rv);
            ptx::tmem_ld_wait();
            uint32_t pe[8], pv[8];
#pragma unroll
            for (int j = 0; j < 8; ++j) {
                float e2[2];
#pragma unroll
                for (int k = 0; k < 2; ++k) {
                    const float z = __uint_as_float(ru[2 * j + k]) - mu;
                    const float gr = fmaf(2.f, ptx::ex2(z * z * nisl2), -1.f);
                    const float a = fminf(fmaxf(gr * __uint_as_float(ri[2 * j + k]), -80.f), 80.f);
                    e2[k] = ptx::ex2(a * LOG2E);
                }
                pe[j] = pack_bf16(e2[0], e2[1]);
                pv[j] = pack_bf16(__uint_as_float(rv[2 * j]), __uint_as_float(rv[2 * j + 1]));
            }
            if (valid_ep) {
                uint4* pE = reinterpret_cast<uint4*>(E + obase + c0);
                uint4* pV = reinterpret_cast<uint4*>(V + obase + c0);
                pE[0] = make_uint4(pe[0], pe[1], pe[2], pe[3]);
                pE[1] = make_uint4(pe[4], pe[5], pe[6], pe[7]);
                pV[0] = make_uint4(pv[0], pv[1], pv[2], pv[3]);
                pV[1] = make_uint4(pv[4], pv[5], pv[6], pv[7]);
            }
        }
        ptx::tc_fence_before();
        __syncthreads();       // TMEM and a_conv are free for the next head
    }
    if (warp == 0) ptx::tmem_dealloc(tmem, k1b::TMEM_COLS);
}

// =============================================================================================================
__global__ void __launch_bounds__(K2B_THREADS, 2)
k2_bf16(const __grid_constant__ CUtensorMap map_wo, __nv_bfloat16* __restrict__ X, const float* __restrict__ scale,
        const __nv_bfloat16* __restrict__ E, const __nv_bfloat16* __restrict__ V, float* __restrict__ partial,
        __nv_bfloat16* __restrict__ vprime, int* __restrict__ status, Geom g) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* sm = align1024(smem_raw);
    uint8_t* a_vp = sm + k2b::A_VP;
    uint8_t* es = sm + k2b::ES;       // [12][20] cells x 128 B
    uint8_t* vs = sm + k2b::VS;       // [10][18] cells x 128 B: V, then R in place
    float* red = reinterpret_cast<float*>(es);   // [128][64] fp32 after the last head
    float* scale_s = reinterpret_cast<float*>(sm + k2b::SCALE);
    uint64_t* full = reinterpret_cast<uint64_t*>(sm + k2b::BARS);
    uint64_t* mma_bar = full + 2;
    uint32_t* tmem_ptr = reinterpret_cast<uint32_t*>(sm + k2b::TMEM_PTR);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int b = blockIdx.y;
    const int tx0 = (blockIdx.x % g.tiles_x) * TBW;
    const int ty0 = (blockIdx.x / g.tiles_x) * TBH;
    const int set = b / g.per_set;
    const size_t xplane = (size_t)g.state_rows() * g.W * NC;
    const size_t eplane = (size_t)g.ev_rows() * g.W * HD;
    const size_t vplane = (size_t)g.H * g.W * HD;

    if (tid == 0) {
        ptx::mbar_init(&full[0], 1);
        ptx::mbar_init(&full[1], 1);
        ptx::mbar_init(mma_bar, 1);
        ptx::fence_barrier_init();
        ptx::prefetch_tmap(&map_wo);
    }
    if (warp == 0) ptx::tmem_alloc(tmem_ptr, k2b::TMEM_COLS);
    if (tid < NC) scale_s[tid] = scale[b * NC + tid];
    ptx::tc_fence_before();
    __syncthreads();
    ptx::tc_fence_after();
    const uint32_t tmem = *tmem_ptr;

    if (tid == 0) {
        for (int s = 0; s < 2; ++s) {
            ptx::mbar_expect_tx(&full[s], k2b::WO_STAGE);
            ptx::tma_load_2d(sm + k2b::WO0 + s * k2b::WO_STAGE, &map_wo, 0, (set * NH + s) * 64, &full[s]);
        }
    }
    const uint32_t idesc = ptx::umma_idesc_bf16(128, 64);

    for (int h = 0; h < NH; ++h) {
        const __nv_bfloat16* Eh = E + ((size_t)b * NH + h) * eplane;
        const __nv_bfloat16* Vh = V + ((size_t)b * NH + h) * eplane;
        for (int i = tid; i < 240 * 8; i += K2B_THREADS) {
            const int q = i & 7, cell = i >> 3;
            const int r = ty0 + cell / 20 - 2, x = g.wrap_x(tx0 + cell % 20 - 2);
            ptx::cp_async16(es + cell * 128 + q * 16, Eh + ((size_t)g.erow(r) * g.W + x) * HD + q * 8);
        }
        for (int i = tid; i < 180 * 8; i += K2B_THREADS) {
            const int q = i & 7, cell = i >> 3;
            const int r = ty0 + cell / 18 - 1, x = g.wrap_x(tx0 + cell % 18 - 1);
            ptx::cp_async16(vs + cell * 128 + q * 16, Vh + ((size_t)g.erow(r) * g.W + x) * HD + q * 8);
        }
        ptx::cp_async_commit();
        ptx::cp_async_wait<0>();
        __syncthreads();

        // ---- R = V / box3(E) on the 10 x 18 ring-extended tile: 18 columns x 8 chunks x 2 row segments ------
        {
            const int q = tid & 7, c = (tid >> 3) % 18, r0 = (tid / 144) * 5;
            float hp2[8], hp1[8];
#pragma unroll
            for (int j = 0; j < 7; ++j) {
                const uint8_t* row = es + ((r0 + j) * 20 + c) * 128 + q * 16;
                float e0[8], e1[8], e2[8], hs[8];
                unpack8(*reinterpret_cast<const uint4*>(row), e0);
                unpack8(*reinterpret_cast<const uint4*>(row + 128), e1);
                unpack8(*reinterpret_cast<const uint4*>(row + 256), e2);
#pragma unroll
                for (int k = 0; k < 8; ++k) hs[k] = (e0[k] + e1[k]) + e2[k];
                if (j >= 2) {
                    uint4* pv = reinterpret_cast<uint4*>(vs + ((r0 + j - 2) * 18 + c) * 128 + q * 16);
                    float v[8];
                    unpack8(*pv, v);
#pragma unroll
                    for (int k = 0; k < 8; ++k) v[k] *= ptx::rcp((hp2[k] + hp1[k]) + hs[k]);
                    *pv = pack8(v);
                }
#pragma unroll
                for (int k = 0; k < 8; ++k) { hp2[k] = hp1[k]; hp1[k] = hs[k]; }
            }
        }
        __syncthreads();
        if (h > 0) {            // the previous head's UMMA must be done reading a_vp and its Wo stage
            ptx::mbar_wait(mma_bar, (h - 1) & 1, status, 201);
            if (tid == 0 && h + 1 < NH) {
                ptx::mbar_expect_tx(&full[(h + 1) & 1], k2b::WO_STAGE);
                ptx::tma_load_2d(sm + k2b::WO0 + ((h + 1) & 1) * k2b::WO_STAGE, &map_wo, 0, (set * NH + h + 1) * 64, &full[(h + 1) & 1]);
            }
        }
        // ---- V' = E * box3(R) on the 8 x 16 tile: 16 columns x 8 chunks x 2 row segments -> A operand ------
        if (tid < 256) {
            const int q = tid & 7, c = (tid >> 3) & 15, r0 = (tid >> 7) * 4;
            float hp2[8], hp1[8];
#pragma unroll
            for (int j = 0; j < 6; ++j) {
                const uint8_t* row = vs + ((r0 + j) * 18 + c) * 128 + q * 16;
                float a0[8], a1[8], a2[8], hs[8];
                unpack8(*reinterpret_cast<const uint4*>(row), a0);
                unpack8(*reinterpret_cast<const uint4*>(row + 128), a1);
                unpack8(*reinterpret_cast<const uint4*>(row + 256), a2);
#pragma unroll
                for (int k = 0; k < 8; ++k) hs[k] = (a0[k] + a1[k]) + a2[k];
                if (j >= 2) {
                    const int orow = r0 + j - 2;
                    float e[8];
                    unpack8(*reinterpret_cast<const uint4*>(es + ((orow + 2) * 20 + c + 2) * 128 + q * 16), e);
#pragma unroll
                    for (int k = 0; k < 8; ++k) e[k] *= (hp2[k] + hp1[k]) + hs[k];
                    const uint4 out = pack8(e);
                    *reinterpret_cast<uint4*>(a_vp + swz(orow * TBW + c, q)) = out;
                    if (vprime != nullptr && ty0 + orow < g.H && tx0 + c < g.W)
                        *reinterpret_cast<uint4*>(vprime + ((size_t)b * NH + h) * vplane +
                                                  ((size_t)(ty0 + orow) * g.W + tx0 + c) * HD + q * 8) = out;
                }
#pragma unroll
                for (int k = 0; k < 8; ++k) { hp2[k] = hp1[k]; hp1[k] = hs[k]; }
            }
        }
        ptx::fence_proxy_async();
        __syncthreads();
        if (tid == 0) {
            ptx::mbar_wait(&full[h & 1], (h >> 1) & 1, status, 202);
            ptx::tc_fence_after();
            const uint64_t da = ptx::umma_desc_sw128(ptx::smem_u32(a_vp));
            const uint64_t dw = ptx::umma_desc_sw128(ptx::smem_u32(sm + k2b::WO0 + (h & 1) * k2b::WO_STAGE));
#pragma unroll
            for (int k = 0; k < 4; ++k) ptx::umma_bf16(tmem, da + 2 * k, dw + 2 * k, idesc, h > 0 || k > 0);
            ptx::umma_commit(mma_bar);
        }
    }
    ptx::mbar_wait(mma_bar, (NH - 1) & 1, status, 203);
    ptx::tc_fence_after();

    // ---- X+ = scale * X + dt * Y (bf16, in place) and the per-channel sums of what was stored -------------------
    if (warp < 8) {
        const int quad = warp & 3, half = warp >> 2;
        const int m = quad * 32 + lane;
        const int r = ty0 + (m >> 4), x = tx0 + (m & 15);
        const bool valid = r < g.H && x < g.W;
        __nv_bfloat16* px = X + (size_t)b * xplane + ((size_t)g.xrow(r) * g.W + (valid ? x : 0)) * NC;
#pragma unroll
        for (int sub = 0; sub < 2; ++sub) {
            const int c0 = half * 32 + sub * 16;
            uint32_t ry[16];
            ptx::tmem_ld16(tmem + ((uint32_t)(quad * 32) << 16) + c0, ry);
            ptx::tmem_ld_wait();
            float xo[16];
            if (valid) {
                float f0[8], f1[8];
                unpack8(*reinterpret_cast<const uint4*>(px + c0), f0);
                unpack8(*reinterpret_cast<const uint4*>(px + c0 + 8), f1);
#pragma unroll
                for (int k = 0; k < 8; ++k) {
                    xo[k] = fmaf(g.dt, __uint_as_float(ry[k]), f0[k] * scale_s[c0 + k]);
                    xo[8 + k] = fmaf(g.dt, __uint_as_float(ry[8 + k]), f1[k] * scale_s[c0 + 8 + k]);
                }
                uint32_t pk[8];
#pragma unroll
                for (int k = 0; k < 8; ++k) {
                    pk[k] = pack_bf16(xo[2 * k], xo[2 * k + 1]);
                    xo[2 * k] = bf16_lo(pk[k]);          // sum what is stored, after rounding
                    xo[2 * k + 1] = bf16_hi(pk[k]);
                }
                *reinterpret_cast<uint4*>(px + c0) = make_uint4(pk[0], pk[1], pk[2], pk[3]);
                *reinterpret_cast<uint4*>(px + c0 + 8) = make_uint4(pk[4], pk[5], pk[6], pk[7]);
            } else {
#pragma unroll
                for (int k = 0; k < 16; ++k) xo[k] = 0.f;
            }
#pragma unroll
            for (int k = 0; k < 16; k += 4)
                *reinterpret_cast<float4*>(red + m * 64 + c0 + k) = make_float4(xo[k], xo[k + 1], xo[k + 2], xo[k + 3]);
        }
    }
    ptx::tc_fence_before();
    __syncthreads();
    if (tid < NC) {
        float t = 0.f;
        for (int m = 0; m < 128; ++m) t += red[m * 64 + tid];
        partial[((size_t)b * gridDim.x + blockIdx.x) * NC + tid] = t;
    }
    if (warp == 0) ptx::tmem_dealloc(tmem, k2b::TMEM_COLS);
}

// =============================================================================================================
// host side
inline const char*& bf16_error_ref() { static const char* e = ""; return e; }
inline const char* bf16_error() { return bf16_error_ref(); }

inline void bf16_plan(Bf16Plan& p, const Geom& g) {
    p.tiles_x = (g.W + TBW - 1) / TBW;
    p.k1_tiles = p.tiles_x * ((g.ev_rows() + TBH - 1) / TBH);
    p.k2_tiles = p.tiles_x * ((g.H + TBH - 1) / TBH);
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

inline int make_weight_map(EncodeTiledFn enc, CUtensorMap* map, const void* base, uint64_t rows, uint32_t box_rows) {
    const cuuint64_t dims[2] = {64, rows};
    const cuuint64_t strides[1] = {128};
    const cuuint32_t box[2] = {64, box_rows};
    const cuuint32_t estr[2] = {1, 1};
    CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(base), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : -1;
}

// Tensor maps over the weight arrays and the kernels' shared-memory opt-in.  Returns 0 on success.
inline int bf16_setup(Bf16Plan& p, const __nv_bfloat16* w1, const __nv_bfloat16* wo, int sets) {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) != cudaSuccess || !fn ||
        q != cudaDriverEntryPointSuccess) {
        bf16_error_ref() = "cuTensorMapEncodeTiled is not available from the driver";
        return -1;
    }
    EncodeTiledFn enc = reinterpret_cast<EncodeTiledFn>(fn);
    if (make_weight_map(enc, &p.map_w1, w1, (uint64_t)sets * NH * 192, 192) ||
        make_weight_map(enc, &p.map_wo, wo, (uint64_t)sets * NH * 64, 64)) {
        bf16_error_ref() = "cuTensorMapEncodeTiled rejected the weight layout";
        return -1;
    }
    if (cudaFuncSetAttribute(k1_bf16, cudaFuncAttributeMaxDynamicSharedMemorySize, k1b::SMEM) != cudaSuccess ||
        cudaFuncSetAttribute(k2_bf16, cudaFuncAttributeMaxDynamicSharedMemorySize, k2b::SMEM) != cudaSuccess) {
        bf16_error_ref() = "could not opt in to the kernels' dynamic shared memory";
        return -1;
    }
    return 0;
}

inline int bf16_k1(Bf16Plan& p, const __nv_bfloat16* X, const float* scale, const float* prm, __nv_bfloat16* E,
                   __nv_bfloat16* V, int* status, const Geom& g, cudaStream_t st) {
    k1_bf16<<<dim3(p.k1_tiles, g.B), K1B_THREADS, k1b::SMEM, st>>>(p.map_w1, X, scale, prm, E, V, status, g);
    return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

inline int bf16_k2(Bf16Plan& p, __nv_bfloat16* X, const float* scale, const __nv_bfloat16* E, const __nv_bfloat16* V,
                   float* partial, __nv_bfloat16* vprime, int* status, const Geom& g, cudaStream_t st) {
    k2_bf16<<<dim3(p.k2_tiles, g.B), K2B_THREADS, k2b::SMEM, st>>>(p.map_wo, X, scale, E, V, partial, vprime, status, g);
    return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

}  // namespace slime
