// bf16 path of the CA step: bf16 storage of state, weights and intermediates, fp32 accumulation and stencil
// math, projections on the 5th-generation tensor cores (tcgen05.mma, accumulators in TMEM, operand tiles
// fetched by TMA).  Same two-kernel split as the fp32 path (ca_f32.cuh):
//
//   k1_bf16  per 8x16-cell tile (128 cells = UMMA M): state halo tile -> per head the 3x3-convolved input as a
//            swizzled K-major A operand; U = conv_h(X) Wp_h (N=64) and I|V = X [Wi_h|Wv_h] (N=128) into 192
//            TMEM columns; epilogue: growth bell, E = exp(G*I), write E and V (bf16, per-head planes).
//   k2_bf16  persistent, warp-specialised, one CTA per SM.  A producer warp streams (tile, head) items - the E
//            tile with a 2-cell halo, the V tile with a 1-cell halo and the head's Wo slice - through a 3-stage
//            TMA ring; two groups of 9 compute warps take alternate heads: separable box sums marching down
//            columns in packed fp32 (R = V / box3(E) in place, V' = E * box3(R)), V' written as a swizzled A
//            operand; an MMA warp issues Y += V'_h Wo_h (N=64) into a double-buffered TMEM accumulator in head
//            order; the epilogue X+ = scale*X + dt*Y (bf16, in place) and the tile's channel sums run one tile
//            behind.
//
// E/V planes are [B][8][H+4][W+4][64] with a 2-cell apron all around: k1 writes every cell it computes to its
// own position and to every apron position that wraps onto it, so k2 never wraps or clamps and each of its
// tiles is one TMA box (boxes hanging over the far edge are zero-filled and only feed cells that are masked).
//
// Shared-memory UMMA operand tiles are [rows][128 B] with the 128-byte swizzle: the 16-byte chunk q of row m
// lives at m*128 + ((q ^ (m & 7)) << 4), tile bases 1024-byte aligned.
#pragma once
#include <cuda.h>

#include "common.cuh"
#include "ptx.cuh"

namespace slime {

constexpr int TBH = 8, TBW = 16;      // tile: 8 rows x 16 columns = 128 cells
constexpr int APRON = 2;              // apron of the E/V planes, cells
constexpr float LOG2E = 1.4426950408889634f;

// Tensor maps k1 stores through: the whole 8 x 16 tile, and - for grids made of whole tiles - the pieces whose
// wrapped copies land at the low end of an apron (a TMA store may hang over the far edge of the tensor, where it
// is clipped, but must not start before its origin): the tile's last two columns, last two rows and their corner.
struct K1StoreMaps {
    CUtensorMap e, v;           // box 64 x 16 x 8 x 1, 128B swizzle
    CUtensorMap e_col, v_col;   // box 64 x 2 x 8 x 1
    CUtensorMap e_row, v_row;   // box 64 x 16 x 2 x 1
    CUtensorMap e_cor, v_cor;   // box 64 x 2 x 2 x 1
};

struct Bf16Plan {
    int tiles_x = 1, k1_tiles = 1, k2_tiles = 1, k1_grid = 1, k2_grid = 1;
    CUtensorMap map_w1;   // [sets*8*192][64] bf16, box 64 x 192, 128B swizzle
    CUtensorMap map_wo;   // [sets*8*64][64]  bf16, box 64 x 64,  128B swizzle
    CUtensorMap map_e;    // E planes [B*8][H+4][W+4][64], box 64 x 20 x 12 x 1
    CUtensorMap map_v;    // V planes, box 64 x 18 x 10 x 1
    K1StoreMaps st;       // store maps of k1 (whole tile, last two columns, last two rows, their corner)
    bool k1_aligned = false;
};

// ---- shared-memory maps (byte offsets from a 1024-aligned base) -------------------------------------------
namespace k1b {
constexpr int A_X = 0;                                   // 2 x 16 KB: X operand of the current / next tile
constexpr int A_CONV = 2 * 16384;                        // 4 x 16 KB: stencil operand slots, two per half
constexpr int W0 = A_CONV + 4 * 16384, W_STAGE = 24576;  // 2 x 24 KB: Wp|Wi|Wv rows of a head
constexpr int STG_E = W0 + 2 * W_STAGE, STG_V = STG_E + 16384;   // staging tiles of the TMA stores
constexpr int STG_COL_E = STG_V + 16384, STG_COL_V = STG_COL_E + 2048;   // last two columns  [8][2] cells
constexpr int STG_ROW_E = STG_COL_V + 2048, STG_ROW_V = STG_ROW_E + 4096; // last two rows     [2][16] cells
constexpr int STG_COR_E = STG_ROW_V + 4096, STG_COR_V = STG_COR_E + 1024; // their corner      [2][2] cells
constexpr int XH = STG_COR_V + 1024, XH_BYTES = 10 * 18 * 128;   // state halo tile, plain [10][18] cells x 128 B
constexpr int PRM_ST = XH + XH_BYTES, PRM_EP = PRM_ST + NH * PRM * 4;   // per-tile copies of the head parameters
constexpr int BARS = PRM_EP + NH * PRM * 4, TMEM_PTR = BARS + 24 * 8;
constexpr int BYTES = TMEM_PTR + 16;
constexpr int SMEM = BYTES + 1024;    // slack for manual 1024-byte alignment
constexpr uint32_t TMEM_COLS = 512;   // two accumulator buffers of 192 columns
constexpr int THREADS = 576;
static_assert(SMEM <= 227 * 1024, "k1 shared memory");
}  // namespace k1b
namespace k2b {
constexpr int STAGES = 3;
constexpr int WO_OFF = 0, E_OFF = 8192, E_BYTES = 12 * 20 * 128, V_OFF = E_OFF + E_BYTES, V_BYTES = 10 * 18 * 128;
constexpr uint32_t STAGE_TX = 8192 + E_BYTES + V_BYTES;                 // 61952 bytes land per item
constexpr int STAGE_BYTES = 62464;                                      // rounded up to a multiple of 1024
constexpr int A_VP = STAGES * STAGE_BYTES;                              // two 16 KB operand tiles, one per group
constexpr int RED = A_VP + 2 * 16384;                                   // [2 groups][4 quads][64] fp32
constexpr int BARS = RED + 2 * 4 * 64 * 4;
constexpr int TMEM_PTR = BARS + 20 * 8;
constexpr int BYTES = TMEM_PTR + 16;
constexpr int SMEM = BYTES + 1024;
constexpr uint32_t TMEM_COLS = 128;                                     // two 64-column accumulators
constexpr int GROUP = 288;                                              // compute threads per group (9 warps)
constexpr int THREADS = 2 * GROUP + 64;                                 // + TMA warp + MMA warp
static_assert(STAGE_TX <= STAGE_BYTES && STAGE_BYTES % 1024 == 0, "stage layout");
static_assert(SMEM <= 227 * 1024, "k2 shared memory");
}  // namespace k2b

__device__ __forceinline__ void unpack8(const uint4& v, float (&f)[8]) {
    f[0] = bf16_lo(v.x); f[1] = bf16_hi(v.x); f[2] = bf16_lo(v.y); f[3] = bf16_hi(v.y);
    f[4] = bf16_lo(v.z); f[5] = bf16_hi(v.z); f[6] = bf16_lo(v.w); f[7] = bf16_hi(v.w);
}
__device__ __forceinline__ uint4 pack8(const float (&f)[8]) {
    return make_uint4(pack_bf16(f[0], f[1]), pack_bf16(f[2], f[3]), pack_bf16(f[4], f[5]), pack_bf16(f[6], f[7]));
}
__device__ __forceinline__ void unpack8p(const uint4& v, ptx::f2 (&f)[4]) {
    f[0] = ptx::bf16x2_to_f2(v.x); f[1] = ptx::bf16x2_to_f2(v.y); f[2] = ptx::bf16x2_to_f2(v.z); f[3] = ptx::bf16x2_to_f2(v.w);
}
__device__ __forceinline__ uint4 pack8p(const ptx::f2 (&f)[4]) {
    return make_uint4(ptx::f2_to_bf16x2(f[0]), ptx::f2_to_bf16x2(f[1]), ptx::f2_to_bf16x2(f[2]), ptx::f2_to_bf16x2(f[3]));
}
__device__ __forceinline__ uint8_t* align1024(uint8_t* p) {
    return reinterpret_cast<uint8_t*>((reinterpret_cast<uintptr_t>(p) + 1023) & ~uintptr_t(1023));
}
__device__ __forceinline__ uint32_t swz(int m, int q) { return (uint32_t)(m * 128 + ((q ^ (m & 7)) << 4)); }

// =============================================================================================================
// A tile of 8 x 16 cells: grid b, origin (ty0, tx0) in own coordinates, linear index over all grids.
struct CaTile {
    int b, ty0, tx0, index;
};
__device__ __forceinline__ CaTile ca_tile(int t, int tiles_per_grid, int tiles_x, int row0) {
    CaTile r;
    r.index = t;
    r.b = t / tiles_per_grid;
    const int tt = t - r.b * tiles_per_grid;
    r.ty0 = (tt / tiles_x) * TBH + row0;
    r.tx0 = (tt % tiles_x) * TBW;
    return r;
}

// k1: persistent, warp-specialised, one CTA per SM (576 threads):
//   warps 0-7   stencil group: loads the tile's state halo (scale applied) and the X operand, then its two
//               4-warp halves take alternate heads: 3x3 stencil marching down columns in packed fp32 -> A operand
//   warps 8-15  epilogue group: TMEM -> growth bell, E = exp(G*I) -> swizzled staging tiles -> TMA store of the
//               whole tile (+ register stores of the apron duplicates of edge cells)
//   warp 16     TMA producer of the per-head weight tiles (2-stage ring)
//   warp 17     UMMA issuer: U (N=64) and I|V (N=128) into a double-buffered 192-column TMEM accumulator
// ALIGNED: the grid is made of whole tiles (W a multiple of 16, and H a multiple of 8 on a torus), so the wrapped
// copies of edge cells are whole pieces of a tile and go out as extra TMA stores; otherwise the threads that own
// edge cells store the copies from registers.
template <bool ALIGNED>
__global__ void __launch_bounds__(k1b::THREADS, 1)
k1_bf16(const __grid_constant__ CUtensorMap map_w1, const __grid_constant__ K1StoreMaps sm_maps,
        const __nv_bfloat16* __restrict__ X,
        const float* __restrict__ scale, const float* __restrict__ prm, __nv_bfloat16* __restrict__ E,
        __nv_bfloat16* __restrict__ V, int* __restrict__ status, int n_tiles, int tiles_per_grid, Geom g) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* sm = align1024(smem_raw);
    uint64_t* bars = reinterpret_cast<uint64_t*>(sm + k1b::BARS);
    // one waiting party per barrier, observing every phase in turn
    uint64_t* w_full = bars;            // [2] weight tile of an item landed             (waits: UMMA issuer)
    uint64_t* w_empty = bars + 3;       // [2] ... and was consumed                      (waits: TMA producer)
    uint64_t* ac_full = bars + 6;       // [4] stencil operand slot written              (waits: UMMA issuer)
    uint64_t* ac_empty = bars + 10;     // [4] ... and consumed                          (waits: the half that owns the slot)
    uint64_t* ax_full = bars + 14;      // [2] X operand of a tile written               (waits: UMMA issuer)
    uint64_t* ax_empty = bars + 16;     // [2] ... all 8 heads of that tile issued+done  (waits: stencil group)
    uint64_t* tm_full = bars + 18;      // [2] accumulator buffer holds an item          (waits: epilogue group)
    uint64_t* tm_empty = bars + 20;     // [2] ... and was drained (256 arrivals)        (waits: UMMA issuer)
    uint32_t* tmem_ptr = reinterpret_cast<uint32_t*>(sm + k1b::TMEM_PTR);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (tid == 0) {
        for (int i = 0; i < 20; ++i) ptx::mbar_init(&bars[i], 1);
        ptx::mbar_init(&tm_empty[0], 256);
        ptx::mbar_init(&tm_empty[1], 256);
        ptx::fence_barrier_init();
        ptx::prefetch_tmap(&map_w1); ptx::prefetch_tmap(&sm_maps.e); ptx::prefetch_tmap(&sm_maps.v);
    }
    if (warp == 0) ptx::tmem_alloc(tmem_ptr, k1b::TMEM_COLS);
    ptx::tc_fence_before();
    __syncthreads();
    ptx::tc_fence_after();
    const uint32_t tmem = *tmem_ptr;
    const int my_tiles = n_tiles > (int)blockIdx.x ? (n_tiles - 1 - (int)blockIdx.x) / (int)gridDim.x + 1 : 0;
    const size_t xplane = (size_t)g.state_rows() * g.W * NC;
    const size_t eplane = (size_t)g.ev_h * g.ev_w * HD;

    if (warp == 16) {
        // ================= TMA producer: weights of item i = (tile k, head h) into stage i % 3 ================
        if (lane == 0) {
            for (int k = 0; k < my_tiles; ++k) {
                const CaTile t = ca_tile(blockIdx.x + k * gridDim.x, tiles_per_grid, g.tiles_x, -g.he);
                const int set = t.b / g.per_set;
                for (int h = 0; h < NH; ++h) {
                    const int i = k * NH + h, ws = i & 1;
                    ptx::mbar_wait(&w_empty[ws], ((i >> 1) & 1) ^ 1, status, 110);
                    ptx::mbar_expect_tx(&w_full[ws], k1b::W_STAGE);
                    ptx::tma_load_2d(sm + k1b::W0 + ws * k1b::W_STAGE, &map_w1, 0, (set * NH + h) * 192, &w_full[ws]);
                }
            }
        }
    } else if (warp == 17) {
        // ================= UMMA issuer =======================================================================
        if (lane == 0) {
            const uint32_t idesc_u = ptx::umma_idesc_bf16(128, 64);
            const uint32_t idesc_iv = ptx::umma_idesc_bf16(128, 128);
            for (int k = 0; k < my_tiles; ++k) {
                const int xb = k & 1;
                for (int h = 0; h < NH; ++h) {
                    const int i = k * NH + h, ws = i & 1, half = h & 1, n = k * 4 + (h >> 1);
                    const int slot = half * 2 + (n & 1), tb = i & 1;
                    if (h == 0) ptx::mbar_wait(&ax_full[xb], (k >> 1) & 1, status, 120);
                    ptx::mbar_wait(&w_full[ws], (i >> 1) & 1, status, 121);
                    ptx::mbar_wait(&ac_full[slot], (n >> 1) & 1, status, 122);
                    ptx::mbar_wait(&tm_empty[tb], ((i >> 1) & 1) ^ 1, status, 123);
                    ptx::tc_fence_after();
                    const uint32_t wb = ptx::smem_u32(sm + k1b::W0 + ws * k1b::W_STAGE);
                    const uint64_t da = ptx::umma_desc_sw128(ptx::smem_u32(sm + k1b::A_CONV + slot * 16384));
                    const uint64_t dx = ptx::umma_desc_sw128(ptx::smem_u32(sm + k1b::A_X + xb * 16384));
                    const uint64_t dwp = ptx::umma_desc_sw128(wb);
                    const uint64_t dwiv = ptx::umma_desc_sw128(wb + 64 * 128);
                    const uint32_t acc = tmem + tb * 192;
#pragma unroll
                    for (int kk = 0; kk < 4; ++kk) ptx::umma_bf16(acc, da + 2 * kk, dwp + 2 * kk, idesc_u, kk > 0);
#pragma unroll
                    for (int kk = 0; kk < 4; ++kk) ptx::umma_bf16(acc + 64, dx + 2 * kk, dwiv + 2 * kk, idesc_iv, kk > 0);
                    ptx::umma_commit(&w_empty[ws]);
                    ptx::umma_commit(&ac_empty[slot]);
                    ptx::umma_commit(&tm_full[tb]);
                    if (h == NH - 1) ptx::umma_commit(&ax_empty[xb]);
                }
            }
        }
    } else if (warp < 8) {
        // ================= stencil group ======================================================================
        const int half = warp >> 2, st = tid & 127;
        uint8_t* xh = sm + k1b::XH;
        float* prm_s = reinterpret_cast<float*>(sm + k1b::PRM_ST);
        for (int k = 0; k < my_tiles; ++k) {
            const CaTile t = ca_tile(blockIdx.x + k * gridDim.x, tiles_per_grid, g.tiles_x, -g.he);
            const int set = t.b / g.per_set;
            uint8_t* a_x = sm + k1b::A_X + (k & 1) * 16384;
            ptx::bar_sync(1, 256);                                        // both halves are done with the last halo
            ptx::mbar_wait(&ax_empty[k & 1], ((k >> 1) & 1) ^ 1, status, 130);
            const float* sc = scale + t.b * NC;
            if (tid < NH * PRM) prm_s[tid] = __ldg(prm + (size_t)set * NH * PRM + tid);
            if (k + 1 < my_tiles && tid < 180) {       // next tile's halo cells: one 128-byte line each, into L2
                const CaTile tn = ca_tile(blockIdx.x + (k + 1) * gridDim.x, tiles_per_grid, g.tiles_x, -g.he);
                const int r = tn.ty0 + tid / 18 - 1, x = g.wrap_x(tn.tx0 + tid % 18 - 1);
                ptx::prefetch_l2(X + (size_t)tn.b * xplane + ((size_t)g.xrow(r) * g.W + x) * NC);
            }
            {
                // 180 cells x 8 chunks over 256 threads: issue every global load first, then scale and store
                const int q = tid & 7;                 // constant per thread: 256 is a multiple of 8
                const float4 s0 = __ldg(reinterpret_cast<const float4*>(sc + q * 8));
                const float4 s1 = __ldg(reinterpret_cast<const float4*>(sc + q * 8 + 4));
                uint4 raw[6];
#pragma unroll
                for (int n = 0; n < 6; ++n) {
                    const int cell = (tid >> 3) + n * 32;
                    if (cell < 180) {
                        const int r = t.ty0 + cell / 18 - 1, x = g.wrap_x(t.tx0 + cell % 18 - 1);
                        raw[n] = *reinterpret_cast<const uint4*>(X + (size_t)t.b * xplane + ((size_t)g.xrow(r) * g.W + x) * NC + q * 8);
                    }
                }
#pragma unroll
                for (int n = 0; n < 6; ++n) {
                    const int cell = (tid >> 3) + n * 32;
                    if (cell < 180) {
                        const int hy = cell / 18, hx = cell % 18;
                        float f[8];
                        unpack8(raw[n], f);
                        f[0] *= s0.x; f[1] *= s0.y; f[2] *= s0.z; f[3] *= s0.w;
                        f[4] *= s1.x; f[5] *= s1.y; f[6] *= s1.z; f[7] *= s1.w;
                        const uint4 v = pack8(f);
                        *reinterpret_cast<uint4*>(xh + cell * 128 + q * 16) = v;
                        if (hy >= 1 && hy <= TBH && hx >= 1 && hx <= TBW)
                            *reinterpret_cast<uint4*>(a_x + swz((hy - 1) * TBW + hx - 1, q)) = v;
                    }
                }
            }
            ptx::fence_proxy_async();
            ptx::bar_sync(1, 256);
            if (tid == 0) ptx::mbar_arrive(&ax_full[k & 1]);

            const int q = st & 7, x = st >> 3;
            for (int h = half; h < NH; h += 2) {
                const int n = k * 4 + (h >> 1), slot = half * 2 + (n & 1);
                uint8_t* a_conv = sm + k1b::A_CONV + slot * 16384;
                ptx::f2 kt[9];
#pragma unroll
                for (int tt = 0; tt < 9; ++tt) { const float kv = prm_s[h * PRM + tt]; kt[tt] = ptx::make_f2(kv, kv); }
                ptx::mbar_wait(&ac_empty[slot], ((n >> 1) & 1) ^ 1, status, 131);
                // input row j feeds output rows j (tap row 0), j-1 (tap row 1) and j-2 (tap row 2)
                ptx::f2 s1[4], s2[4];
#pragma unroll
                for (int j = 0; j < 10; ++j) {
                    const uint8_t* row = xh + (j * 18 + x) * 128 + q * 16;
                    ptx::f2 c0[4], c1[4], c2[4], nw[4], md[4];
                    unpack8p(*reinterpret_cast<const uint4*>(row), c0);
                    unpack8p(*reinterpret_cast<const uint4*>(row + 128), c1);
                    unpack8p(*reinterpret_cast<const uint4*>(row + 256), c2);
                    if (j >= 2) {
                        ptx::f2 o[4];
#pragma unroll
                        for (int e = 0; e < 4; ++e)
                            o[e] = ptx::fma2(kt[6], c0[e], ptx::fma2(kt[7], c1[e], ptx::fma2(kt[8], c2[e], s2[e])));
                        *reinterpret_cast<uint4*>(a_conv + swz((j - 2) * TBW + x, q)) = pack8p(o);
                    }
                    if (j >= 1 && j <= 8) {
#pragma unroll
                        for (int e = 0; e < 4; ++e)
                            md[e] = ptx::fma2(kt[3], c0[e], ptx::fma2(kt[4], c1[e], ptx::fma2(kt[5], c2[e], s1[e])));
                    }
                    if (j <= 7) {
#pragma unroll
                        for (int e = 0; e < 4; ++e)
                            nw[e] = ptx::fma2(kt[0], c0[e], ptx::fma2(kt[1], c1[e], ptx::mul2(kt[2], c2[e])));
                    }
#pragma unroll
                    for (int e = 0; e < 4; ++e) { s2[e] = md[e]; s1[e] = nw[e]; }
                }
                ptx::fence_proxy_async();
                ptx::bar_sync(2 + half, 128);
                if (st == 0) ptx::mbar_arrive(&ac_full[slot]);
            }
        }
    } else {
        // ================= epilogue group (warps 8..15) ========================================================
        const int et = tid - 256, quad = warp & 3, half = (warp - 8) >> 2;
        const int m_ep = quad * 32 + lane;                 // TMEM lane = cell of the tile this thread finishes
        uint8_t* stg_e = sm + k1b::STG_E;
        uint8_t* stg_v = sm + k1b::STG_V;
        float* prm_e = reinterpret_cast<float*>(sm + k1b::PRM_EP);
        const bool tiny = g.W < 2 * APRON || (g.wrap_y && g.H < 2 * APRON);
        for (int k = 0; k < my_tiles; ++k) {
            const CaTile t = ca_tile(blockIdx.x + k * gridDim.x, tiles_per_grid, g.tiles_x, -g.he);
            const int set = t.b / g.per_set;
            const int r_ep = t.ty0 + (m_ep >> 4), x_ep = t.tx0 + (m_ep & 15);
            const bool valid_ep = r_ep < g.H + g.he && x_ep < g.W;
            ptx::bar_sync(4, 256);                     // everyone is done with the last tile's parameters
            if (et < NH * PRM) prm_e[et] = __ldg(prm + (size_t)set * NH * PRM + et);
            ptx::bar_sync(4, 256);
            // Apron positions that wrap onto this thread's cell (the TMA store below covers the cell itself and
            // whatever hangs over the far edge).
            const int cy = m_ep >> 4, cx = m_ep & 15;
            // whole-tile grids: which sides of the grid this tile touches (uniform over the tile)
            const bool left = t.tx0 == 0, right = t.tx0 + TBW == g.W;
            const bool top = g.wrap_y && t.ty0 == 0, bottom = g.wrap_y && t.ty0 + TBH == g.H;
            const bool in_col = right && cx >= TBW - APRON, in_row = bottom && cy >= TBH - APRON;
            // ragged or tiny grids: per-thread targets (named registers, not an indexed array: an array would live
            // in local memory and put a load in front of every duplicate store).  Grids narrower or shorter than
            // twice the apron can wrap more than once and take the general loop.
            size_t off_x = 0, off_y = 0, off_xy = 0;
            bool dup_x = false, dup_y = false;
            if (!ALIGNED && valid_ep && !tiny) {
                const int xd = x_ep < APRON ? x_ep + g.W : (x_ep >= g.W - APRON ? x_ep - g.W : -100);
                const int rd = !g.wrap_y ? -100 : (r_ep < APRON ? r_ep + g.H : (r_ep >= g.H - APRON ? r_ep - g.H : -100));
                dup_x = xd != -100;
                dup_y = rd != -100;
                if (dup_x) off_x = ((size_t)(r_ep + APRON) * g.ev_w + xd + APRON) * HD;
                if (dup_y) off_y = ((size_t)(rd + APRON) * g.ev_w + x_ep + APRON) * HD;
                if (dup_x && dup_y) off_xy = ((size_t)(rd + APRON) * g.ev_w + xd + APRON) * HD;
            }
            const bool any_dup = !ALIGNED && valid_ep && (dup_x || dup_y || tiny);
            for (int h = 0; h < NH; ++h) {
                const int i = k * NH + h, tb = i & 1;
                const float mus = prm_e[h * PRM + 9];            // mu * s; Wp carries s and Wi carries log2(e)
                const ptx::f2 neg_mus2 = ptx::make_f2(-mus, -mus), two2 = ptx::make_f2(2.f, 2.f), minus_one2 = ptx::make_f2(-1.f, -1.f);
                ptx::mbar_wait(&tm_full[tb], (i >> 1) & 1, status, 140);
                ptx::tc_fence_after();
                const uint32_t t_lane = tmem + ((uint32_t)(quad * 32) << 16) + tb * 192;
                uint32_t pe[2][8], pv[2][8];
#pragma unroll
                for (int sub = 0; sub < 2; ++sub) {
                    const int c0 = half * 32 + sub * 16;
                    uint32_t ru[16], ri[16], rv[16];
                    ptx::tmem_ld16(t_lane + c0, ru);
                    ptx::tmem_ld16(t_lane + 64 + c0, ri);
                    ptx::tmem_ld16(t_lane + 128 + c0, rv);
                    ptx::tmem_ld_wait();
#pragma unroll
                    for (int j = 0; j < 8; ++j) {
                        // two elements at a time in packed fp32; only the two ex2 and the clamp are per element
                        const ptx::f2 z = ptx::add2(ptx::make_f2(__uint_as_float(ru[2 * j]), __uint_as_float(ru[2 * j + 1])), neg_mus2);
                        float q0, q1;
                        ptx::split_f2(ptx::mul2(z, z), q0, q1);
                        const ptx::f2 gr = ptx::fma2(ptx::make_f2(ptx::ex2(-q0), ptx::ex2(-q1)), two2, minus_one2);
                        float a0, a1;
                        ptx::split_f2(ptx::mul2(gr, ptx::make_f2(__uint_as_float(ri[2 * j]), __uint_as_float(ri[2 * j + 1]))), a0, a1);
                        pe[sub][j] = pack_bf16(ptx::ex2(fminf(fmaxf(a0, -ACT_CLAMP * LOG2E), ACT_CLAMP * LOG2E)),
                                               ptx::ex2(fminf(fmaxf(a1, -ACT_CLAMP * LOG2E), ACT_CLAMP * LOG2E)));
                        pv[sub][j] = pack_bf16(__uint_as_float(rv[2 * j]), __uint_as_float(rv[2 * j + 1]));
                    }
                }
                ptx::tc_fence_before();
                ptx::mbar_arrive(&tm_empty[tb]);                  // the accumulator buffer is free again
                if (et == 0) ptx::bulk_wait_read0();              // the last TMA stores are done reading the staging
                ptx::bar_sync(4, 256);
#pragma unroll
                for (int sub = 0; sub < 2; ++sub) {
                    const int qa = half * 4 + sub * 2;
                    const uint4 e_lo = make_uint4(pe[sub][0], pe[sub][1], pe[sub][2], pe[sub][3]);
                    const uint4 e_hi = make_uint4(pe[sub][4], pe[sub][5], pe[sub][6], pe[sub][7]);
                    const uint4 v_lo = make_uint4(pv[sub][0], pv[sub][1], pv[sub][2], pv[sub][3]);
                    const uint4 v_hi = make_uint4(pv[sub][4], pv[sub][5], pv[sub][6], pv[sub][7]);
                    *reinterpret_cast<uint4*>(stg_e + swz(m_ep, qa)) = e_lo;
                    *reinterpret_cast<uint4*>(stg_e + swz(m_ep, qa + 1)) = e_hi;
                    *reinterpret_cast<uint4*>(stg_v + swz(m_ep, qa)) = v_lo;
                    *reinterpret_cast<uint4*>(stg_v + swz(m_ep, qa + 1)) = v_hi;
                    if (ALIGNED) {
                        if (in_col) {
                            const int mc = cy * APRON + cx - (TBW - APRON);
                            *reinterpret_cast<uint4*>(sm + k1b::STG_COL_E + swz(mc, qa)) = e_lo;
                            *reinterpret_cast<uint4*>(sm + k1b::STG_COL_E + swz(mc, qa + 1)) = e_hi;
                            *reinterpret_cast<uint4*>(sm + k1b::STG_COL_V + swz(mc, qa)) = v_lo;
                            *reinterpret_cast<uint4*>(sm + k1b::STG_COL_V + swz(mc, qa + 1)) = v_hi;
                        }
                        if (in_row) {
                            const int mr = (cy - (TBH - APRON)) * TBW + cx;
                            *reinterpret_cast<uint4*>(sm + k1b::STG_ROW_E + swz(mr, qa)) = e_lo;
                            *reinterpret_cast<uint4*>(sm + k1b::STG_ROW_E + swz(mr, qa + 1)) = e_hi;
                            *reinterpret_cast<uint4*>(sm + k1b::STG_ROW_V + swz(mr, qa)) = v_lo;
                            *reinterpret_cast<uint4*>(sm + k1b::STG_ROW_V + swz(mr, qa + 1)) = v_hi;
                        }
                        if (in_col && in_row) {
                            const int mq = (cy - (TBH - APRON)) * APRON + cx - (TBW - APRON);
                            *reinterpret_cast<uint4*>(sm + k1b::STG_COR_E + swz(mq, qa)) = e_lo;
                            *reinterpret_cast<uint4*>(sm + k1b::STG_COR_E + swz(mq, qa + 1)) = e_hi;
                            *reinterpret_cast<uint4*>(sm + k1b::STG_COR_V + swz(mq, qa)) = v_lo;
                            *reinterpret_cast<uint4*>(sm + k1b::STG_COR_V + swz(mq, qa + 1)) = v_hi;
                        }
                    }
                    if (any_dup) {
                        __nv_bfloat16* Eh = E + ((size_t)t.b * NH + h) * eplane + half * 32 + sub * 16;
                        __nv_bfloat16* Vh = V + ((size_t)t.b * NH + h) * eplane + half * 32 + sub * 16;
                        if (!tiny) {
                            if (dup_x) {
                                uint4* pE = reinterpret_cast<uint4*>(Eh + off_x);
                                uint4* pV = reinterpret_cast<uint4*>(Vh + off_x);
                                pE[0] = e_lo; pE[1] = e_hi; pV[0] = v_lo; pV[1] = v_hi;
                            }
                            if (dup_y) {
                                uint4* pE = reinterpret_cast<uint4*>(Eh + off_y);
                                uint4* pV = reinterpret_cast<uint4*>(Vh + off_y);
                                pE[0] = e_lo; pE[1] = e_hi; pV[0] = v_lo; pV[1] = v_hi;
                            }
                            if (dup_x && dup_y) {
                                uint4* pE = reinterpret_cast<uint4*>(Eh + off_xy);
                                uint4* pV = reinterpret_cast<uint4*>(Vh + off_xy);
                                pE[0] = e_lo; pE[1] = e_hi; pV[0] = v_lo; pV[1] = v_hi;
                            }
                        } else {
                            for (int ky = -2 * APRON; ky <= 2 * APRON; ++ky)
                                for (int kx = -2 * APRON; kx <= 2 * APRON; ++kx) {
                                    if ((ky != 0 && !g.wrap_y) || (ky == 0 && kx == 0)) continue;
                                    const int rr = r_ep + ky * g.H, xx = x_ep + kx * g.W;
                                    if (rr < -APRON || rr >= g.H + APRON || xx < -APRON || xx >= g.W + APRON) continue;
                                    const size_t off = ((size_t)(rr + APRON) * g.ev_w + xx + APRON) * HD;
                                    uint4* pE = reinterpret_cast<uint4*>(Eh + off);
                                    uint4* pV = reinterpret_cast<uint4*>(Vh + off);
                                    pE[0] = e_lo; pE[1] = e_hi; pV[0] = v_lo; pV[1] = v_hi;
                                }
                        }
                    }
                }
                ptx::fence_proxy_async();
                ptx::bar_sync(4, 256);
                if (et == 0) {
                    const int px = t.tx0 + APRON, py = t.ty0 + APRON, pl = t.b * NH + h;
                    ptx::tma_store_4d(&sm_maps.e, stg_e, 0, px, py, pl);
                    ptx::tma_store_4d(&sm_maps.v, stg_v, 0, px, py, pl);
                    if (ALIGNED) {
                        // wrapped copies: pieces that land at the high end of an apron are the whole tile stored at the
                        // shifted position (all but the first two columns / rows are clipped); pieces that land at
                        // the low end come from the small staging tiles
                        const int hx = g.W + APRON, hy = g.H + APRON;
                        if (left) { ptx::tma_store_4d(&sm_maps.e, stg_e, 0, hx, py, pl); ptx::tma_store_4d(&sm_maps.v, stg_v, 0, hx, py, pl); }
                        if (top) { ptx::tma_store_4d(&sm_maps.e, stg_e, 0, px, hy, pl); ptx::tma_store_4d(&sm_maps.v, stg_v, 0, px, hy, pl); }
                        if (left && top) { ptx::tma_store_4d(&sm_maps.e, stg_e, 0, hx, hy, pl); ptx::tma_store_4d(&sm_maps.v, stg_v, 0, hx, hy, pl); }
                        if (right) {
                            ptx::tma_store_4d(&sm_maps.e_col, sm + k1b::STG_COL_E, 0, 0, py, pl);
                            ptx::tma_store_4d(&sm_maps.v_col, sm + k1b::STG_COL_V, 0, 0, py, pl);
                            if (top) {
                                ptx::tma_store_4d(&sm_maps.e_col, sm + k1b::STG_COL_E, 0, 0, hy, pl);
                                ptx::tma_store_4d(&sm_maps.v_col, sm + k1b::STG_COL_V, 0, 0, hy, pl);
                            }
                        }
                        if (bottom) {
                            ptx::tma_store_4d(&sm_maps.e_row, sm + k1b::STG_ROW_E, 0, px, 0, pl);
                            ptx::tma_store_4d(&sm_maps.v_row, sm + k1b::STG_ROW_V, 0, px, 0, pl);
                            if (left) {
                                ptx::tma_store_4d(&sm_maps.e_row, sm + k1b::STG_ROW_E, 0, hx, 0, pl);
                                ptx::tma_store_4d(&sm_maps.v_row, sm + k1b::STG_ROW_V, 0, hx, 0, pl);
                            }
                            if (right) {
                                ptx::tma_store_4d(&sm_maps.e_cor, sm + k1b::STG_COR_E, 0, 0, 0, pl);
                                ptx::tma_store_4d(&sm_maps.v_cor, sm + k1b::STG_COR_V, 0, 0, 0, pl);
                            }
                        }
                    }
                    ptx::bulk_commit();
                }
            }
        }
        if (et == 0) ptx::bulk_wait0();
    }
    ptx::tc_fence_before();
    __syncthreads();
    if (warp == 0) ptx::tmem_dealloc(tmem, k1b::TMEM_COLS);
}

// =============================================================================================================

// Epilogue of one finished tile, run by 8 warps (256 threads) of one compute group: X+ = scale*X + dt*Y in
// place, and the tile's per-channel sums of the stored (rounded) values -> partial[tile][64].
__device__ __forceinline__ void k2_epilogue(const CaTile& t, uint32_t acc_taddr, __nv_bfloat16* __restrict__ X,
                                            const float* __restrict__ scale, float* __restrict__ partial,
                                            float* red, int bar_id, int gt, int cta_warp, const Geom& g) {
    const int lane = gt & 31, quad = cta_warp & 3, half = (gt >> 5) >> 2;
    const int m = quad * 32 + lane;
    const int r = t.ty0 + (m >> 4), x = t.tx0 + (m & 15);
    const bool valid = r < g.H && x < g.W;
    const size_t xplane = (size_t)g.state_rows() * g.W * NC;
    __nv_bfloat16* px = X + (size_t)t.b * xplane + ((size_t)g.xrow(valid ? r : 0) * g.W + (valid ? x : 0)) * NC;
    const float* sc = scale + t.b * NC;
#pragma unroll
    for (int sub = 0; sub < 2; ++sub) {
        const int c0 = half * 32 + sub * 16;
        uint32_t ry[16];
        ptx::tmem_ld16(acc_taddr + ((uint32_t)(quad * 32) << 16) + c0, ry);
        ptx::tmem_ld_wait();
        float xo[16];
        if (valid) {
            float f0[8], f1[8], sv[16];
            unpack8(*reinterpret_cast<const uint4*>(px + c0), f0);
            unpack8(*reinterpret_cast<const uint4*>(px + c0 + 8), f1);
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const float4 s4 = __ldg(reinterpret_cast<const float4*>(sc + c0) + k);
                sv[4 * k] = s4.x; sv[4 * k + 1] = s4.y; sv[4 * k + 2] = s4.z; sv[4 * k + 3] = s4.w;
            }
#pragma unroll
            for (int k = 0; k < 8; ++k) {
                xo[k] = fmaf(g.dt, __uint_as_float(ry[k]), f0[k] * sv[k]);
                xo[8 + k] = fmaf(g.dt, __uint_as_float(ry[8 + k]), f1[k] * sv[8 + k]);
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
        // sum over the 32 cells of this warp, fixed tree: each step halves the channels a lane carries
#pragma unroll
        for (int w = 8; w >= 1; w >>= 1) {
            const bool up = (lane & (w * 2)) != 0;
#pragma unroll
            for (int j = 0; j < w; ++j) {
                const float send = up ? xo[j] : xo[j + w];
                const float keep = up ? xo[j + w] : xo[j];
                xo[j] = keep + __shfl_xor_sync(0xffffffffu, send, w * 2);
            }
        }
        xo[0] += __shfl_xor_sync(0xffffffffu, xo[0], 1);
        if ((lane & 1) == 0) {
            const int ch = ((lane >> 4) & 1) * 8 + ((lane >> 3) & 1) * 4 + ((lane >> 2) & 1) * 2 + ((lane >> 1) & 1);
            red[quad * 64 + c0 + ch] = xo[0];
        }
    }
    ptx::bar_sync(bar_id, 256);
    if (gt < NC) partial[(size_t)t.index * NC + gt] = (red[gt] + red[64 + gt]) + (red[128 + gt] + red[192 + gt]);
}

__global__ void __launch_bounds__(k2b::THREADS, 1)
k2_bf16(const __grid_constant__ CUtensorMap map_wo, const __grid_constant__ CUtensorMap map_e,
        const __grid_constant__ CUtensorMap map_v, __nv_bfloat16* __restrict__ X, const float* __restrict__ scale,
        float* __restrict__ partial, __nv_bfloat16* __restrict__ vprime, int* __restrict__ status, int n_tiles,
        int tiles_per_grid, Geom g) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* sm = align1024(smem_raw);
    uint64_t* bars = reinterpret_cast<uint64_t*>(sm + k2b::BARS);
    // Every barrier has exactly one waiting party that observes each of its phases in turn (a parity wait can
    // not tell a phase from the one two earlier).  Items alternate between the two compute groups and between
    // three stages, so "TMA landed" is kept per (group, stage): item i uses full[(i & 1) * 3 + i % 3], phase i / 6.
    uint64_t* full = bars;              // [2][3] TMA landed in stage s for group g
    uint64_t* empty = bars + 6;         // [3]  the UMMA of the item in stage s is done (Wo read; E/V long since)
    uint64_t* vp_full = bars + 9;       // [2]  group g's operand tile is written
    uint64_t* vp_empty = bars + 11;     // [2]  the UMMA reading group g's operand tile is done
    uint64_t* acc_full = bars + 13;     // [2]  all 8 heads of a tile are accumulated
    uint64_t* acc_empty = bars + 15;    // [2]  the epilogue has drained the accumulator
    uint32_t* tmem_ptr = reinterpret_cast<uint32_t*>(sm + k2b::TMEM_PTR);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (tid == 0) {
        for (int i = 0; i < 6; ++i) ptx::mbar_init(&full[i], 1);
        for (int i = 0; i < 3; ++i) ptx::mbar_init(&empty[i], 1);
        for (int i = 0; i < 2; ++i) {
            ptx::mbar_init(&vp_full[i], 1); ptx::mbar_init(&vp_empty[i], 1);
            ptx::mbar_init(&acc_full[i], 1); ptx::mbar_init(&acc_empty[i], 256);
        }
        ptx::fence_barrier_init();
        ptx::prefetch_tmap(&map_wo); ptx::prefetch_tmap(&map_e); ptx::prefetch_tmap(&map_v);
    }
    if (warp == 0) ptx::tmem_alloc(tmem_ptr, k2b::TMEM_COLS);
    ptx::tc_fence_before();
    __syncthreads();
    ptx::tc_fence_after();
    const uint32_t tmem = *tmem_ptr;
    const int my_tiles = n_tiles > (int)blockIdx.x ? (n_tiles - 1 - (int)blockIdx.x) / (int)gridDim.x + 1 : 0;

    if (warp == 18) {
        // ================= TMA producer ===================================================================
        if (lane == 0) {
            for (int k = 0; k < my_tiles; ++k) {
                const CaTile t = ca_tile(blockIdx.x + k * gridDim.x, tiles_per_grid, g.tiles_x, 0);
                const int set = t.b / g.per_set;
                for (int h = 0; h < NH; ++h) {
                    const int i = k * NH + h, s = i % 3, u = i / 3;
                    ptx::mbar_wait(&empty[s], (u & 1) ^ 1, status, 210);
                    uint8_t* st = sm + s * k2b::STAGE_BYTES;
                    uint64_t* fb = &full[(h & 1) * 3 + s];
                    ptx::mbar_expect_tx(fb, k2b::STAGE_TX);
                    ptx::tma_load_2d(st + k2b::WO_OFF, &map_wo, 0, (set * NH + h) * 64, fb);
                    ptx::tma_load_4d(st + k2b::E_OFF, &map_e, 0, t.tx0, t.ty0, t.b * NH + h, fb);
                    ptx::tma_load_4d(st + k2b::V_OFF, &map_v, 0, t.tx0 + 1, t.ty0 + 1, t.b * NH + h, fb);
                    // pull the item three ahead into L2 while this one streams into shared memory
                    const int j = i + 3, kj = j / NH, hj = j % NH;
                    if (kj < my_tiles) {
                        const CaTile tj = ca_tile(blockIdx.x + kj * gridDim.x, tiles_per_grid, g.tiles_x, 0);
                        ptx::tma_prefetch_4d(&map_e, 0, tj.tx0, tj.ty0, tj.b * NH + hj);
                        ptx::tma_prefetch_4d(&map_v, 0, tj.tx0 + 1, tj.ty0 + 1, tj.b * NH + hj);
                    }
                }
            }
        }
    } else if (warp == 19) {
        // ================= UMMA issuer ====================================================================
        if (lane == 0) {
            const uint32_t idesc = ptx::umma_idesc_bf16(128, 64);
            for (int k = 0; k < my_tiles; ++k) {
                const int ab = k & 1, w = k >> 1;
                for (int h = 0; h < NH; ++h) {
                    const int i = k * NH + h, s = i % 3, grp = h & 1, v = i >> 1;
                    if (h == 0) ptx::mbar_wait(&acc_empty[ab], (w & 1) ^ 1, status, 220);
                    ptx::mbar_wait(&full[grp * 3 + s], (i / 6) & 1, status, 221);
                    ptx::mbar_wait(&vp_full[grp], v & 1, status, 222);
                    ptx::tc_fence_after();
                    const uint64_t da = ptx::umma_desc_sw128(ptx::smem_u32(sm + k2b::A_VP + grp * 16384));
                    const uint64_t dw = ptx::umma_desc_sw128(ptx::smem_u32(sm + s * k2b::STAGE_BYTES + k2b::WO_OFF));
#pragma unroll
                    for (int kk = 0; kk < 4; ++kk)
                        ptx::umma_bf16(tmem + ab * 64, da + 2 * kk, dw + 2 * kk, idesc, h > 0 || kk > 0);
                    ptx::umma_commit(&empty[s]);
                    ptx::umma_commit(&vp_empty[grp]);
                    if (h == NH - 1) ptx::umma_commit(&acc_full[ab]);
                }
            }
        }
    } else {
        // ================= compute groups: group 0 = warps 0..8 takes even heads, group 1 = warps 9..17 odd ====
        const int grp = warp >= 9 ? 1 : 0;
        const int gt = tid - grp * k2b::GROUP;          // 0..287 inside the group
        const int bar_main = 1 + grp, bar_ep = 3 + grp;
        uint8_t* a_vp = sm + k2b::A_VP + grp * 16384;
        float* red = reinterpret_cast<float*>(sm + k2b::RED) + grp * 256;
        const size_t vplane = (size_t)g.H * g.W * HD;
        CaTile prev;
        prev.index = -1;
        for (int k = 0; k < my_tiles; ++k) {
            const CaTile t = ca_tile(blockIdx.x + k * gridDim.x, tiles_per_grid, g.tiles_x, 0);
            for (int h = grp; h < NH; h += 2) {
                const int i = k * NH + h, s = i % 3, v = i >> 1;
                uint8_t* es = sm + s * k2b::STAGE_BYTES + k2b::E_OFF;   // [12][20] cells x 128 B
                uint8_t* vs = sm + s * k2b::STAGE_BYTES + k2b::V_OFF;   // [10][18] cells x 128 B: V, then R in place
                ptx::mbar_wait(&full[grp * 3 + s], (i / 6) & 1, status, 230);

                // ---- R = V / box3(E) on the 10 x 18 ring-extended tile: 18 columns x 8 chunks x 2 row segments ----
                {
                    const int q = gt & 7, c = (gt >> 3) % 18, r0 = (gt / 144) * 5;
                    ptx::f2 hp2[4], hp1[4];
#pragma unroll
                    for (int j = 0; j < 7; ++j) {
                        const uint8_t* row = es + ((r0 + j) * 20 + c) * 128 + q * 16;
                        const uint4 e0 = *reinterpret_cast<const uint4*>(row);
                        const uint4 e1 = *reinterpret_cast<const uint4*>(row + 128);
                        const uint4 e2 = *reinterpret_cast<const uint4*>(row + 256);
                        ptx::f2 hs[4];
                        hs[0] = ptx::sum3_bf16x2(e0.x, e1.x, e2.x); hs[1] = ptx::sum3_bf16x2(e0.y, e1.y, e2.y);
                        hs[2] = ptx::sum3_bf16x2(e0.z, e1.z, e2.z); hs[3] = ptx::sum3_bf16x2(e0.w, e1.w, e2.w);
                        if (j >= 2) {
                            uint4* pv = reinterpret_cast<uint4*>(vs + ((r0 + j - 2) * 18 + c) * 128 + q * 16);
                            ptx::f2 vv[4];
                            unpack8p(*pv, vv);
#pragma unroll
                            for (int n = 0; n < 4; ++n) {
                                float z0, z1;
                                ptx::split_f2(ptx::add2(ptx::add2(hp2[n], hp1[n]), hs[n]), z0, z1);
                                vv[n] = ptx::mul2(vv[n], ptx::make_f2(ptx::rcp(z0), ptx::rcp(z1)));
                            }
                            *pv = pack8p(vv);
                        }
#pragma unroll
                        for (int n = 0; n < 4; ++n) { hp2[n] = hp1[n]; hp1[n] = hs[n]; }
                    }
                }
                ptx::bar_sync(bar_main, k2b::GROUP);
                ptx::mbar_wait(&vp_empty[grp], (v & 1) ^ 1, status, 231);   // the UMMA two heads back is done with a_vp

                // ---- V' = E * box3(R) on the 8 x 16 tile: 16 columns x 8 chunks x 2 row segments -> A operand ----
                if (gt < 256) {
                    const int q = gt & 7, c = (gt >> 3) & 15, r0 = (gt >> 7) * 4;
                    ptx::f2 hp2[4], hp1[4];
#pragma unroll
                    for (int j = 0; j < 6; ++j) {
                        const uint8_t* row = vs + ((r0 + j) * 18 + c) * 128 + q * 16;
                        const uint4 a0 = *reinterpret_cast<const uint4*>(row);
                        const uint4 a1 = *reinterpret_cast<const uint4*>(row + 128);
                        const uint4 a2 = *reinterpret_cast<const uint4*>(row + 256);
                        ptx::f2 hs[4];
                        hs[0] = ptx::sum3_bf16x2(a0.x, a1.x, a2.x); hs[1] = ptx::sum3_bf16x2(a0.y, a1.y, a2.y);
                        hs[2] = ptx::sum3_bf16x2(a0.z, a1.z, a2.z); hs[3] = ptx::sum3_bf16x2(a0.w, a1.w, a2.w);
                        if (j >= 2) {
                            const int orow = r0 + j - 2;
                            ptx::f2 e[4];
                            unpack8p(*reinterpret_cast<const uint4*>(es + ((orow + 2) * 20 + c + 2) * 128 + q * 16), e);
#pragma unroll
                            for (int n = 0; n < 4; ++n) e[n] = ptx::mul2(e[n], ptx::add2(ptx::add2(hp2[n], hp1[n]), hs[n]));
                            const uint4 out = pack8p(e);
                            *reinterpret_cast<uint4*>(a_vp + swz(orow * TBW + c, q)) = out;
                            if (vprime != nullptr && t.ty0 + orow < g.H && t.tx0 + c < g.W)
                                *reinterpret_cast<uint4*>(vprime + ((size_t)t.b * NH + h) * vplane +
                                                          ((size_t)(t.ty0 + orow) * g.W + t.tx0 + c) * HD + q * 8) = out;
                        }
#pragma unroll
                        for (int n = 0; n < 4; ++n) { hp2[n] = hp1[n]; hp1[n] = hs[n]; }
                    }
                }
                ptx::fence_proxy_async();
                ptx::bar_sync(bar_main, k2b::GROUP);
                if (gt == 0) ptx::mbar_arrive(&vp_full[grp]);

                // ---- epilogue of the previous tile, one tile behind, by the group of that tile's parity --------
                if (h == 2 + grp && prev.index >= 0 && ((k - 1) & 1) == grp && gt < 256) {
                    const int pk = k - 1, ab = pk & 1, w = pk >> 1;
                    ptx::mbar_wait(&acc_full[ab], w & 1, status, 232);
                    ptx::tc_fence_after();
                    k2_epilogue(prev, tmem + ab * 64, X, scale, partial, red, bar_ep, gt, warp, g);
                    ptx::tc_fence_before();
                    ptx::mbar_arrive(&acc_empty[ab]);
                }
            }
            prev = t;
        }
        if (my_tiles > 0 && ((my_tiles - 1) & 1) == grp && gt < 256) {
            const int pk = my_tiles - 1, ab = pk & 1, w = pk >> 1;
            ptx::mbar_wait(&acc_full[ab], w & 1, status, 233);
            ptx::tc_fence_after();
            k2_epilogue(prev, tmem + ab * 64, X, scale, partial, red, bar_ep, gt, warp, g);
            ptx::tc_fence_before();
            ptx::mbar_arrive(&acc_empty[ab]);
        }
    }
    ptx::tc_fence_before();
    __syncthreads();
    if (warp == 0) ptx::tmem_dealloc(tmem, k2b::TMEM_COLS);
}

// =============================================================================================================
// host side
inline const char*& bf16_error_ref() { static const char* e = ""; return e; }
inline const char* bf16_error() { return bf16_error_ref(); }

inline void bf16_plan(Bf16Plan& p, const Geom& g) {
    p.tiles_x = (g.W + TBW - 1) / TBW;
    p.k1_tiles = p.tiles_x * ((g.H + 2 * g.he + TBH - 1) / TBH);
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

// Tile map over the E or V planes: [planes][ev_h][ev_w][64] bf16, box 64 x box_w x box_h x 1, no swizzle.
inline int make_plane_map(EncodeTiledFn enc, CUtensorMap* map, const void* base, const Geom& g, uint32_t box_w, uint32_t box_h,
                          CUtensorMapSwizzle swizzle = CU_TENSOR_MAP_SWIZZLE_NONE) {
    const cuuint64_t dims[4] = {64, (cuuint64_t)g.ev_w, (cuuint64_t)g.ev_h, (cuuint64_t)g.B * NH};
    const cuuint64_t strides[3] = {128, (cuuint64_t)g.ev_w * 128, (cuuint64_t)g.ev_h * g.ev_w * 128};
    const cuuint32_t box[4] = {64, box_w, box_h, 1};
    const cuuint32_t estr[4] = {1, 1, 1, 1};
    CUresult r = enc(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<void*>(base), dims, strides, box, estr,
                     CU_TENSOR_MAP_INTERLEAVE_NONE, swizzle, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                     CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    return r == CUDA_SUCCESS ? 0 : -1;
}

// Tensor maps over the weight arrays and the E/V planes, and the kernels' shared-memory opt-in.  0 on success.
inline int bf16_setup(Bf16Plan& p, const __nv_bfloat16* w1, const __nv_bfloat16* wo, int sets, const __nv_bfloat16* E,
                      const __nv_bfloat16* V, const Geom& g, int num_sms) {
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
    if (make_plane_map(enc, &p.map_e, E, g, TBW + 4, TBH + 4) || make_plane_map(enc, &p.map_v, V, g, TBW + 2, TBH + 2) ||
        make_plane_map(enc, &p.st.e, E, g, TBW, TBH, CU_TENSOR_MAP_SWIZZLE_128B) ||
        make_plane_map(enc, &p.st.v, V, g, TBW, TBH, CU_TENSOR_MAP_SWIZZLE_128B) ||
        make_plane_map(enc, &p.st.e_col, E, g, APRON, TBH, CU_TENSOR_MAP_SWIZZLE_128B) ||
        make_plane_map(enc, &p.st.v_col, V, g, APRON, TBH, CU_TENSOR_MAP_SWIZZLE_128B) ||
        make_plane_map(enc, &p.st.e_row, E, g, TBW, APRON, CU_TENSOR_MAP_SWIZZLE_128B) ||
        make_plane_map(enc, &p.st.v_row, V, g, TBW, APRON, CU_TENSOR_MAP_SWIZZLE_128B) ||
        make_plane_map(enc, &p.st.e_cor, E, g, APRON, APRON, CU_TENSOR_MAP_SWIZZLE_128B) ||
        make_plane_map(enc, &p.st.v_cor, V, g, APRON, APRON, CU_TENSOR_MAP_SWIZZLE_128B)) {
        bf16_error_ref() = "cuTensorMapEncodeTiled rejected the E/V plane layout";
        return -1;
    }
    p.k1_aligned = g.W % TBW == 0 && (!g.wrap_y || g.H % TBH == 0);
    if (cudaFuncSetAttribute(k1_bf16<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, k1b::SMEM) != cudaSuccess ||
        cudaFuncSetAttribute(k1_bf16<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, k1b::SMEM) != cudaSuccess ||
        cudaFuncSetAttribute(k2_bf16, cudaFuncAttributeMaxDynamicSharedMemorySize, k2b::SMEM) != cudaSuccess) {
        bf16_error_ref() = "could not opt in to the kernels' dynamic shared memory";
        return -1;
    }
    const long long total = (long long)p.k2_tiles * g.B, total1 = (long long)p.k1_tiles * g.B;
    p.k2_grid = (int)(total < num_sms ? total : num_sms);
    p.k1_grid = (int)(total1 < num_sms ? total1 : num_sms);
    return 0;
}

inline int bf16_k1(Bf16Plan& p, const __nv_bfloat16* X, const float* scale, const float* prm, __nv_bfloat16* E,
                   __nv_bfloat16* V, int* status, const Geom& g, cudaStream_t st) {
    if (p.k1_aligned)
        k1_bf16<true><<<p.k1_grid, k1b::THREADS, k1b::SMEM, st>>>(p.map_w1, p.st, X, scale, prm, E, V, status,
                                                                  p.k1_tiles * g.B, p.k1_tiles, g);
    else
        k1_bf16<false><<<p.k1_grid, k1b::THREADS, k1b::SMEM, st>>>(p.map_w1, p.st, X, scale, prm, E, V, status,
                                                                   p.k1_tiles * g.B, p.k1_tiles, g);
    return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

inline int bf16_k2(Bf16Plan& p, __nv_bfloat16* X, const float* scale, const __nv_bfloat16*, const __nv_bfloat16*,
                   float* partial, __nv_bfloat16* vprime, int* status, const Geom& g, cudaStream_t st) {
    k2_bf16<<<p.k2_grid, k2b::THREADS, k2b::SMEM, st>>>(p.map_wo, p.map_e, p.map_v, X, scale, partial, vprime, status,
                                                        p.k2_tiles * g.B, p.k2_tiles, g);
    return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

}  // namespace slime
