// bf16 path of the CA step: bf16 storage of state, weights and intermediates, fp32 accumulation and stencil
// math, projections on the 5th-generation tensor cores (tcgen05.mma, accumulators in TMEM, operand tiles
// fetched by TMA).  Same two-kernel split as the fp32 path (ca_f32.cuh):
//
//   k1_bf16  per 8x16-cell tile (128 cells = UMMA M): state halo tile -> per head the 3x3-convolved input as a
//            swizzled K-major A operand; U = conv_h(X) Wp_h (N=64) and I|V = X [Wi_h|Wv_h] (N=128) into 192
//            TMEM columns; epilogue: growth bell, E = exp(G*I), write E and V (bf16, per-head planes).
//   k2_bf16  persistent, warp-specialised, one CTA per SM: macro tiles of 32 columns, marched four rows at a time
//            per head with the box sums' vertical running sums carried in registers; R = V / box3(E) and
//            V' = E * box3(R) on two sets of warps one block apart, V' written as a swizzled A operand; an MMA warp
//            issues Y += V'_h Wo_h (N=64) into one TMEM accumulator per 4 x 32-cell tile in head order; the epilogue
//            X+ = scale*X + dt*Y (bf16, in place) and the tiles' channel sums run one macro tile behind.
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
    CUtensorMap map_e;    // E planes [B*8][H+4][W+4][64], box 64 x 36 x 4 x 1 (a block of k2)
    CUtensorMap map_v;    // V planes, box 64 x 34 x 4 x 1
    CUtensorMap map_x;    // the state's own rows (and the halo rows above them) [B][hx + H][W][64], box 64 x 32 x 4 x 1, 128B swizzle
    K1StoreMaps st;       // store maps of k1 (whole tile, last two columns, last two rows, their corner)
    bool k1_aligned = false;
    int strips = 1, mt_per_grid = 1, nbmax = 8;    // k2: 32-column strips, macro tiles per grid, blocks per macro tile
};

// ---- shared-memory maps (byte offsets from a 1024-aligned base) -------------------------------------------
namespace k1b {
constexpr int A_X = 0;                                   // 16 KB: X operand of the current tile
constexpr int A_CONV = 16384;                            // 4 x 16 KB: stencil operand slots, two per half
constexpr int W0 = A_CONV + 4 * 16384, W_STAGE = 24576;  // 2 x 24 KB: Wp|Wi|Wv rows of a head
constexpr int STG_E = W0 + 2 * W_STAGE, STG_V = STG_E + 16384;   // staging tiles of the TMA stores
constexpr int STG_COL_E = STG_V + 16384, STG_COL_V = STG_COL_E + 2048;   // last two columns  [8][2] cells
constexpr int STG_ROW_E = STG_COL_V + 2048, STG_ROW_V = STG_ROW_E + 4096; // last two rows     [2][16] cells
constexpr int STG_COR_E = STG_ROW_V + 4096, STG_COR_V = STG_COR_E + 1024; // their corner      [2][2] cells
constexpr int XH = STG_COR_V + 1024, XH_BYTES = 10 * 18 * 256;   // state halo tile, plain [10][18] cells x 64 fp32
constexpr int PRM_ST = XH + XH_BYTES;                    // per-tile copy of the head parameters (stencil taps)
constexpr int BARS = PRM_ST + NH * PRM * 4, TMEM_PTR = BARS + 24 * 8;
constexpr int BYTES = TMEM_PTR + 16;
constexpr int SMEM = BYTES + 1024;    // slack for manual 1024-byte alignment
constexpr uint32_t TMEM_COLS = 512;   // two accumulator buffers of 192 columns
constexpr int THREADS = 608;
static_assert(SMEM <= 227 * 1024, "k1 shared memory");
}  // namespace k1b

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

// k1: persistent, warp-specialised, one CTA per SM (608 threads):
//   warps 0-7   stencil group: loads the tile's state halo (scale applied) and the X operand, then its two
//               4-warp halves take alternate heads: 3x3 stencil marching down columns in packed fp32 -> A operand
//   warps 8-15  epilogue group: TMEM -> growth bell, E = exp(G*I) -> swizzled staging tiles (+ register stores of
//               the apron duplicates of edge cells on ragged grids)
//   warp 16     TMA producer of the per-head weight tiles (2-stage ring)
//   warp 17     UMMA issuer: U (N=64) and I|V (N=128) into a double-buffered 192-column TMEM accumulator
//   warp 18     store warp: issues the TMA stores of every finished item, so that the epilogue group never meets at
//               a barrier (its threads arrive on an mbarrier when their staging is written and move on)
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
    uint64_t* ax_full = bars + 14;      // X operand of a tile written                   (waits: UMMA issuer)
    uint64_t* ax_empty = bars + 16;     // ... all 8 heads of that tile issued+done      (waits: stencil group)
    uint64_t* tm_full = bars + 18;      // [2] accumulator buffer holds an item          (waits: epilogue group)
    uint64_t* tm_empty = bars + 20;     // [2] ... and was drained (256 arrivals)        (waits: UMMA issuer)
    uint64_t* stg_full = bars + 22;     // staging tiles of an item written (256 arrivals) (waits: store warp)
    uint64_t* stg_free = bars + 23;     // ... and read by the item's TMA stores         (waits: epilogue group)
    uint32_t* tmem_ptr = reinterpret_cast<uint32_t*>(sm + k1b::TMEM_PTR);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (tid == 0) {
        for (int i = 0; i < 20; ++i) ptx::mbar_init(&bars[i], 1);
        ptx::mbar_init(&tm_empty[0], 256);
        ptx::mbar_init(&tm_empty[1], 256);
        ptx::mbar_init(stg_full, 256);
        ptx::mbar_init(stg_free, 1);
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
                for (int h = 0; h < NH; ++h) {
                    const int i = k * NH + h, ws = i & 1, half = h & 1, n = k * 4 + (h >> 1);
                    const int slot = half * 2 + (n & 1), tb = i & 1;
                    if (h == 0) ptx::mbar_wait(ax_full, k & 1, status, 120);
                    ptx::mbar_wait(&w_full[ws], (i >> 1) & 1, status, 121);
                    ptx::mbar_wait(&ac_full[slot], (n >> 1) & 1, status, 122);
                    ptx::mbar_wait(&tm_empty[tb], ((i >> 1) & 1) ^ 1, status, 123);
                    ptx::tc_fence_after();
                    const uint32_t wb = ptx::smem_u32(sm + k1b::W0 + ws * k1b::W_STAGE);
                    const uint64_t da = ptx::umma_desc_sw128(ptx::smem_u32(sm + k1b::A_CONV + slot * 16384));
                    const uint64_t dx = ptx::umma_desc_sw128(ptx::smem_u32(sm + k1b::A_X));
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
                    if (h == NH - 1) ptx::umma_commit(ax_empty);
                }
            }
        }
    } else if (warp == 18) {
        // ================= store warp: the TMA stores of every finished item ==================================
        // The epilogue group never meets at a barrier: its threads arrive on stg_full when their part of the staging
        // tiles is written and go on to the next item; this thread issues the item's stores and hands the staging
        // back (stg_free) as soon as the stores have read it.
        if (lane == 0) {
            for (int k = 0; k < my_tiles; ++k) {
                const CaTile t = ca_tile(blockIdx.x + k * gridDim.x, tiles_per_grid, g.tiles_x, -g.he);
                // whole-tile grids: which sides of the grid this tile touches
                const bool left = t.tx0 == 0, right = t.tx0 + TBW == g.W;
                const bool top = g.wrap_y && t.ty0 == 0, bottom = g.wrap_y && t.ty0 + TBH == g.H;
                for (int h = 0; h < NH; ++h) {
                    const int i = k * NH + h;
                    ptx::mbar_wait(stg_full, i & 1, status, 150);
                    const int px = t.tx0 + APRON, py = t.ty0 + APRON, pl = t.b * NH + h;
                    ptx::tma_store_4d(&sm_maps.e, sm + k1b::STG_E, 0, px, py, pl);
                    ptx::tma_store_4d(&sm_maps.v, sm + k1b::STG_V, 0, px, py, pl);
                    if (ALIGNED) {
                        // wrapped copies: pieces that land at the high end of an apron are the whole tile stored at the
                        // shifted position (all but the first two columns / rows are clipped); pieces that land at
                        // the low end come from the small staging tiles
                        const int hx = g.W + APRON, hy = g.H + APRON;
                        if (left) { ptx::tma_store_4d(&sm_maps.e, sm + k1b::STG_E, 0, hx, py, pl); ptx::tma_store_4d(&sm_maps.v, sm + k1b::STG_V, 0, hx, py, pl); }
                        if (top) { ptx::tma_store_4d(&sm_maps.e, sm + k1b::STG_E, 0, px, hy, pl); ptx::tma_store_4d(&sm_maps.v, sm + k1b::STG_V, 0, px, hy, pl); }
                        if (left && top) { ptx::tma_store_4d(&sm_maps.e, sm + k1b::STG_E, 0, hx, hy, pl); ptx::tma_store_4d(&sm_maps.v, sm + k1b::STG_V, 0, hx, hy, pl); }
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
                    ptx::bulk_wait_read0();
                    ptx::mbar_arrive(stg_free);
                }
            }
            ptx::bulk_wait0();
        }
    } else if (warp < 8) {
        // ================= stencil group ======================================================================
        const int half = warp >> 2, st = tid & 127;
        uint8_t* xh = sm + k1b::XH;
        float* prm_s = reinterpret_cast<float*>(sm + k1b::PRM_ST);
        for (int k = 0; k < my_tiles; ++k) {
            const CaTile t = ca_tile(blockIdx.x + k * gridDim.x, tiles_per_grid, g.tiles_x, -g.he);
            const int set = t.b / g.per_set;
            uint8_t* a_x = sm + k1b::A_X;
            ptx::bar_sync(1, 256);                                        // both halves are done with the last halo
            const float* sc = scale + t.b * NC;
            if (tid < NH * PRM) prm_s[tid] = __ldg(prm + (size_t)set * NH * PRM + tid);
            if (k + 1 < my_tiles && tid < 180) {       // next tile's halo cells: one 128-byte line each, into L2
                const CaTile tn = ca_tile(blockIdx.x + (k + 1) * gridDim.x, tiles_per_grid, g.tiles_x, -g.he);
                const int r = tn.ty0 + tid / 18 - 1, x = g.wrap_x(tn.tx0 + tid % 18 - 1);
                ptx::prefetch_l2(X + (size_t)tn.b * xplane + ((size_t)g.xrow(r) * g.W + x) * NC);
            }
            {
                // 180 cells x 8 chunks over 256 threads: issue every global load first, then scale, round to bf16
                // (the value both operands are made of) and store: fp32 to the halo tile, bf16 to the X operand
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
                // the X operand is single-buffered: the last tile's products have long been issued by the time the
                // loads above come back
                ptx::mbar_wait(ax_empty, (k & 1) ^ 1, status, 130);
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
                        unpack8(v, f);
                        float4* dst = reinterpret_cast<float4*>(xh + cell * 256 + q * 32);
                        dst[0] = make_float4(f[0], f[1], f[2], f[3]);
                        dst[1] = make_float4(f[4], f[5], f[6], f[7]);
                        if (hy >= 1 && hy <= TBH && hx >= 1 && hx <= TBW)
                            *reinterpret_cast<uint4*>(a_x + swz((hy - 1) * TBW + hx - 1, q)) = v;
                    }
                }
            }
            ptx::fence_proxy_async();
            ptx::bar_sync(1, 256);
            if (tid == 0) ptx::mbar_arrive(ax_full);

            // a thread owns two adjacent columns x 4 channels: a row of the halo is four 16-byte loads (cells
            // 2p .. 2p+3), shared by the two outputs, and nothing is unpacked
            const int c4 = st & 15, p2 = st >> 4;
            for (int h = half; h < NH; h += 2) {
                const int n = k * 4 + (h >> 1), slot = half * 2 + (n & 1);
                uint8_t* a_conv = sm + k1b::A_CONV + slot * 16384;
                ptx::f2 kt[9];
#pragma unroll
                for (int tt = 0; tt < 9; ++tt) { const float kv = prm_s[h * PRM + tt]; kt[tt] = ptx::make_f2(kv, kv); }
                ptx::mbar_wait(&ac_empty[slot], ((n >> 1) & 1) ^ 1, status, 131);
                // input row j feeds output rows j (tap row 0), j-1 (tap row 1) and j-2 (tap row 2)
                ptx::f2 s1[2][2], s2[2][2];
#pragma unroll
                for (int j = 0; j < 10; ++j) {
                    const uint8_t* row = xh + (j * 18 + 2 * p2) * 256 + c4 * 16;
                    ptx::f2 c[4][2];
#pragma unroll
                    for (int i = 0; i < 4; ++i) {
                        const float4 w = *reinterpret_cast<const float4*>(row + i * 256);
                        c[i][0] = ptx::make_f2(w.x, w.y);
                        c[i][1] = ptx::make_f2(w.z, w.w);
                    }
#pragma unroll
                    for (int col = 0; col < 2; ++col) {
                        ptx::f2 nw[2], md[2];
                        if (j >= 2) {
                            ptx::f2 o[2];
#pragma unroll
                            for (int e = 0; e < 2; ++e)
                                o[e] = ptx::fma2(kt[6], c[col][e], ptx::fma2(kt[7], c[col + 1][e], ptx::fma2(kt[8], c[col + 2][e], s2[col][e])));
                            *reinterpret_cast<uint2*>(a_conv + swz((j - 2) * TBW + 2 * p2 + col, c4 >> 1) + (c4 & 1) * 8) =
                                make_uint2(ptx::f2_to_bf16x2(o[0]), ptx::f2_to_bf16x2(o[1]));
                        }
                        if (j >= 1 && j <= 8) {
#pragma unroll
                            for (int e = 0; e < 2; ++e)
                                md[e] = ptx::fma2(kt[3], c[col][e], ptx::fma2(kt[4], c[col + 1][e], ptx::fma2(kt[5], c[col + 2][e], s1[col][e])));
                        }
                        if (j <= 7) {
#pragma unroll
                            for (int e = 0; e < 2; ++e)
                                nw[e] = ptx::fma2(kt[0], c[col][e], ptx::fma2(kt[1], c[col + 1][e], ptx::mul2(kt[2], c[col + 2][e])));
                        }
#pragma unroll
                        for (int e = 0; e < 2; ++e) { s2[col][e] = md[e]; s1[col][e] = nw[e]; }
                    }
                }
                ptx::fence_proxy_async();
                ptx::bar_sync(2 + half, 128);
                if (st == 0) ptx::mbar_arrive(&ac_full[slot]);
            }
        }
    } else {
        // ================= epilogue group (warps 8..15) ========================================================
        const int quad = warp & 3, half = (warp - 8) >> 2;
        const int m_ep = quad * 32 + lane;                 // TMEM lane = cell of the tile this thread finishes
        uint8_t* stg_e = sm + k1b::STG_E;
        uint8_t* stg_v = sm + k1b::STG_V;
        const bool tiny = g.W < 2 * APRON || (g.wrap_y && g.H < 2 * APRON);
        for (int k = 0; k < my_tiles; ++k) {
            const CaTile t = ca_tile(blockIdx.x + k * gridDim.x, tiles_per_grid, g.tiles_x, -g.he);
            const int set = t.b / g.per_set;
            const int r_ep = t.ty0 + (m_ep >> 4), x_ep = t.tx0 + (m_ep & 15);
            const bool valid_ep = r_ep < g.H + g.he && x_ep < g.W;
            // Apron positions that wrap onto this thread's cell (the store warp's TMA store covers the cell itself
            // and whatever hangs over the far edge).
            const int cy = m_ep >> 4, cx = m_ep & 15;
            // whole-tile grids: does this tile touch the right / bottom side of the grid (uniform over the tile)
            const bool right = t.tx0 + TBW == g.W, bottom = g.wrap_y && t.ty0 + TBH == g.H;
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
                const float mus = __ldg(prm + ((size_t)set * NH + h) * PRM + 9);   // mu * s; Wp carries s and Wi carries log2(e)
                const ptx::f2 neg_mus2 = ptx::make_f2(-mus, -mus), two2 = ptx::make_f2(2.f, 2.f), minus_one2 = ptx::make_f2(-1.f, -1.f);
                // clamp(G*I) before the exponential = clamp of the rounded exponential (rounding to bf16 is monotone):
                // two packed bf16 min/max per pair instead of four fp32 ones
                const uint32_t e_max = pack_bf16(ptx::ex2(ACT_CLAMP * LOG2E), ptx::ex2(ACT_CLAMP * LOG2E));
                const uint32_t e_min = pack_bf16(ptx::ex2(-ACT_CLAMP * LOG2E), ptx::ex2(-ACT_CLAMP * LOG2E));
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
                        pe[sub][j] = ptx::max_bf16x2(ptx::min_bf16x2(pack_bf16(ptx::ex2(a0), ptx::ex2(a1)), e_max), e_min);
                        pv[sub][j] = pack_bf16(__uint_as_float(rv[2 * j]), __uint_as_float(rv[2 * j + 1]));
                    }
                }
                ptx::tc_fence_before();
                ptx::mbar_arrive(&tm_empty[tb]);                  // the accumulator buffer is free again
                ptx::mbar_wait(stg_free, (i & 1) ^ 1, status, 141);   // the last item's TMA stores are done reading the staging
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
                ptx::mbar_arrive(stg_full);                       // the store warp takes it from here
            }
        }
    }
    ptx::tc_fence_before();
    __syncthreads();
    if (warp == 0) ptx::tmem_dealloc(tmem, k1b::TMEM_COLS);
}

// =============================================================================================================

// Epilogue of one finished tile, run by 8 warps (256 threads) of one compute group: X+ = scale*X + dt*Y in
// place, and the tile's per-channel sums of the stored (rounded) values -> partial[tile][64].
// Epilogue of a finished 4 x 32-cell tile (cell m of the tile = TMEM lane m), by 8 warps (256 threads): X+ = scale*X +
// dt*Y, and the tile's per-channel sums of the stored (rounded) values -> partial[tile][64].  The tile's state sits in
// shared memory, [128 cells][128 B] with the 128-byte swizzle, where a TMA load put it; X+ is written back in place
// and leaves by a TMA store, so the warps never wait on global memory here.
__device__ __forceinline__ void k2_epilogue(const CaTile& t, uint32_t acc_taddr, uint8_t* xs,
                                            const float* __restrict__ scale, float* __restrict__ partial,
                                            float* red, int bar_id, int gt, int cta_warp, const Geom& g) {
    const int lane = gt & 31, quad = cta_warp & 3, half = (gt >> 5) >> 2;
    const int m = quad * 32 + lane;
    const int r = t.ty0 + (m >> 5), x = t.tx0 + (m & 31);
    const bool valid = r < g.H && x < g.W;       // cells outside the grid: loaded as zeros, clipped by the store
    const float* sc = scale + t.b * NC;
#pragma unroll
    for (int sub = 0; sub < 2; ++sub) {
        const int c0 = half * 32 + sub * 16, q0 = half * 4 + sub * 2;
        uint32_t ry[16];
        ptx::tmem_ld16(acc_taddr + ((uint32_t)(quad * 32) << 16) + c0, ry);
        ptx::tmem_ld_wait();
        float xo[16];
        if (valid) {
            float f0[8], f1[8], sv[16];
            uint4* p0 = reinterpret_cast<uint4*>(xs + swz(m, q0));
            uint4* p1 = reinterpret_cast<uint4*>(xs + swz(m, q0 + 1));
            unpack8(*p0, f0);
            unpack8(*p1, f1);
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
            *p0 = make_uint4(pk[0], pk[1], pk[2], pk[3]);
            *p1 = make_uint4(pk[4], pk[5], pk[6], pk[7]);
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
    ptx::fence_proxy_async();      // X+ in shared memory, for the TMA store issued behind the barrier
    ptx::bar_sync(bar_id, 256);
    if (gt < NC) partial[(size_t)t.index * NC + gt] = (red[gt] + red[64 + gt]) + (red[128 + gt] + red[192 + gt]);
}

// =============================================================================================================
// k2.  The grid is cut into macro tiles of 32 columns x 32 rows; a macro tile is eight 4 x 32-cell tiles (UMMA
// M = 128) stacked in y, one 64-column TMEM accumulator each (8 x 64 = all 512 columns; launches with too few macro
// tiles to fill the GPU use 4, 2 or 1 tiles per macro tile instead).  For one head
// after the other the kernel marches down the macro tile four rows at a time, carrying the vertical running sums of
// both box sums in registers from block to block, so every E and V row of the strip is loaded and summed once per
// head (square tiles with a 2-cell ring all round re-read 1.9x the E rows and 1.4x the V rows at 8 x 16 cells).  A
// block is 4 rows of the strip: E rows with a 2-column ring (36 cells), V rows with a 1-column ring (34 cells), 35 KB,
// in a 4-stage ring.  Block -1 of a march only primes the registers (E rows -2..1, R rows -1..0 of the macro tile).
// The two box sums run on different warps, one block apart, with no barrier inside either set:
//   warps 0-7,19 A: R = V / box3(E) in place in the stage, one thread per (column of the 34, 8 dims); hands the block
//                to B through a named barrier it only arrives on
//   warps 8-15   B: V' = E * box3(R) -> one of two swizzled A operand tiles (every thread arrives on the operand's
//                mbarrier), then releases the stage
//   warp 16      TMA producer: per (macro tile, head) the head's Wo slice (double-buffered), per block E and V
//   warp 17      UMMA issuer: Y[tile] += V'_h Wo_h, heads in order
//   warp 18      TMA producer of the epilogues' state tiles (a wait for a free buffer never holds back E / V)
// so that each of the SM's four schedulers (warp index mod 4) carries two A warps and two B warps, the half-filled
// ninth A warp sits alone on the fourth, and the three single-thread roles on the first three.
// The epilogue of a macro tile (X+ = scale X + dt Y, channel sums) is interleaved into the first head of the next one:
// A's first eight warps drain the even accumulators, B the odd ones, each just before its own block of that tile.  The
// tile's state comes to the draining set by TMA (each set owns one 16 KB buffer, refilled as soon as it is free) and X+ leaves
// by a TMA store from the same buffer.
// Every cell's arithmetic is the same sequence of operations wherever the cell sits in a tile or a block, so shifting a
// torus shifts the result bit for bit.
// Eight fp32 values (the 8 dims a thread owns) as four packed pairs, and the few operations the box sums need on them
// (add / mul.f32x2; a plain-fp32 version of the same operations measured 4 % slower).
struct V8 { ptx::f2 v[4]; };
__device__ __forceinline__ V8 v8_zero() { V8 r; for (int i = 0; i < 4; ++i) r.v[i] = ptx::make_f2(0.f, 0.f); return r; }
__device__ __forceinline__ V8 v8_sum3(const uint4& a, const uint4& b, const uint4& c) {
    V8 r;
    r.v[0] = ptx::sum3_bf16x2(a.x, b.x, c.x); r.v[1] = ptx::sum3_bf16x2(a.y, b.y, c.y);
    r.v[2] = ptx::sum3_bf16x2(a.z, b.z, c.z); r.v[3] = ptx::sum3_bf16x2(a.w, b.w, c.w);
    return r;
}
__device__ __forceinline__ V8 v8_add(const V8& a, const V8& b) { V8 r; for (int i = 0; i < 4; ++i) r.v[i] = ptx::add2(a.v[i], b.v[i]); return r; }
__device__ __forceinline__ V8 v8_mul(const V8& a, const V8& b) { V8 r; for (int i = 0; i < 4; ++i) r.v[i] = ptx::mul2(a.v[i], b.v[i]); return r; }
__device__ __forceinline__ V8 v8_rcp(const V8& a) {
    V8 r;
    for (int i = 0; i < 4; ++i) { float z0, z1; ptx::split_f2(a.v[i], z0, z1); r.v[i] = ptx::make_f2(ptx::rcp(z0), ptx::rcp(z1)); }
    return r;
}
__device__ __forceinline__ V8 v8_unpack(const uint4& w) { V8 r; unpack8p(w, r.v); return r; }
__device__ __forceinline__ uint4 v8_pack(const V8& a) { return pack8p(a.v); }

namespace k2m {
constexpr int SW = 32, BR = 4, NB = 8;                  // strip width, rows per block, blocks per macro tile
constexpr int MTH = BR * NB;                            // macro tile height
constexpr int EW = SW + 4, VW = SW + 2;                 // cells per E / V row of a block
constexpr int E_BYTES = BR * EW * 128, V_BYTES = BR * VW * 128;
constexpr int STAGE_BYTES = E_BYTES + V_BYTES;          // 35 840
constexpr uint32_t STAGE_TX = STAGE_BYTES;
constexpr int NSTAGE = 4;
constexpr int STG = 0;
constexpr int A_VP = STG + NSTAGE * STAGE_BYTES;        // two 16 KB operand tiles
constexpr int WO = A_VP + 2 * 16384;                    // two 8 KB Wo slices
constexpr int XT = WO + 2 * 8192;                       // two 16 KB state tiles of the epilogue (one per box-sum set)
constexpr int RED = XT + 2 * 16384;                     // [A, B][4 quads][64] fp32
constexpr int BARS = RED + 2 * 4 * 64 * 4;
constexpr int N_BARS = NSTAGE + NSTAGE + 2 + 2 + 2 + 2 + NB + NB + 2 + 2;
constexpr int TMEM_PTR = BARS + N_BARS * 8;
constexpr int BYTES = TMEM_PTR + 16;
constexpr int SMEM = BYTES + 1024;
constexpr uint32_t TMEM_COLS = 512;
constexpr int A_THREADS = 288, B_THREADS = 256;
constexpr int THREADS = 640;                            // 20 warps, see the kernel for who does what
constexpr int HANDOFF = A_THREADS + B_THREADS;          // parties of the named barrier that hands a block from A to B
static_assert(STAGE_BYTES % 1024 == 0 && A_VP % 1024 == 0 && WO % 1024 == 0 && XT % 1024 == 0, "swizzled tiles must be 1024-byte aligned");
static_assert(SMEM <= 227 * 1024, "k2 (marching) shared memory");
}  // namespace k2m

// Macro tile `idx` of the launch: grid, origin, number of 4-row blocks that hold own rows.
struct MacroTile {
    int b, mx0, my0, nb, tile0;     // tile0: index of its first 4 x 32 tile among the grid's partial sums
};
// nbmax: blocks per full macro tile of this launch (8, 4, 2 or 1)
__device__ __forceinline__ MacroTile macro_tile(int idx, int per_grid, int strips, int H, int nbmax) {
    MacroTile m;
    m.b = idx / per_grid;
    const int r = idx - m.b * per_grid, my = r / strips, sx = r - my * strips;
    m.mx0 = sx * k2m::SW;
    m.my0 = my * nbmax * k2m::BR;
    const int left = (H - m.my0 + k2m::BR - 1) / k2m::BR;
    m.nb = left < nbmax ? left : nbmax;
    m.tile0 = (my * nbmax) * strips + sx;         // tile (block row y4, strip sx) has index y4 * strips + sx
    return m;
}

__global__ void __launch_bounds__(k2m::THREADS, 1)
k2_bf16(const __grid_constant__ CUtensorMap map_wo, const __grid_constant__ CUtensorMap map_e,
              const __grid_constant__ CUtensorMap map_v, const __grid_constant__ CUtensorMap map_x, const float* __restrict__ scale,
              float* __restrict__ partial, __nv_bfloat16* __restrict__ vprime, int* __restrict__ status, int n_mt,
              int mt_per_grid, int strips, int tiles_per_grid, int nbmax, Geom g) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* sm = align1024(smem_raw);
    uint64_t* bars = reinterpret_cast<uint64_t*>(sm + k2m::BARS);
    uint64_t* full = bars;                           // [5] block landed                              (waits: A)
    uint64_t* empty = full + k2m::NSTAGE;            // [5] B is done with the stage (256 arrivals)   (waits: TMA producer)
    uint64_t* vp_full = empty + k2m::NSTAGE;         // [2] operand tile written (256 arrivals)       (waits: UMMA issuer)
    uint64_t* vp_empty = vp_full + 2;                // [2] the UMMAs reading it are done             (waits: B)
    uint64_t* wo_full = vp_empty + 2;                // [2] Wo slice landed                           (waits: UMMA issuer)
    uint64_t* wo_empty = wo_full + 2;                // [2] the head that used it is issued and done  (waits: TMA producer)
    uint64_t* acc_full = wo_empty + 2;               // [8] all 8 heads of the tile accumulated       (waits: who drains it)
    uint64_t* acc_empty = acc_full + k2m::NB;        // [8] drained (256 arrivals)                    (waits: UMMA issuer)
    uint64_t* x_full = acc_empty + k2m::NB;          // [2] a set's state tile landed                 (waits: that set)
    uint64_t* x_empty = x_full + 2;                  // [2] ... and its X+ has left shared memory      (waits: TMA producer)
    uint32_t* tmem_ptr = reinterpret_cast<uint32_t*>(sm + k2m::TMEM_PTR);

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    if (tid == 0) {
        // (every thread of a set arrives by itself: one arrival per warp behind a __syncwarp measured 3 % slower)
        for (int i = 0; i < k2m::NSTAGE; ++i) { ptx::mbar_init(&full[i], 1); ptx::mbar_init(&empty[i], k2m::B_THREADS); }
        for (int i = 0; i < 2; ++i) {
            ptx::mbar_init(&vp_full[i], k2m::B_THREADS); ptx::mbar_init(&vp_empty[i], 1);
            ptx::mbar_init(&wo_full[i], 1); ptx::mbar_init(&wo_empty[i], 1);
        }
        for (int i = 0; i < k2m::NB; ++i) { ptx::mbar_init(&acc_full[i], 1); ptx::mbar_init(&acc_empty[i], 256); }
        for (int i = 0; i < 2; ++i) { ptx::mbar_init(&x_full[i], 1); ptx::mbar_init(&x_empty[i], 1); }
        ptx::fence_barrier_init();
        ptx::prefetch_tmap(&map_wo); ptx::prefetch_tmap(&map_e); ptx::prefetch_tmap(&map_v); ptx::prefetch_tmap(&map_x);
    }
    if (warp == 0) ptx::tmem_alloc(tmem_ptr, k2m::TMEM_COLS);
    ptx::tc_fence_before();
    __syncthreads();
    ptx::tc_fence_after();
    const uint32_t tmem = *tmem_ptr;
    const int my_mt = n_mt > (int)blockIdx.x ? (n_mt - 1 - (int)blockIdx.x) / (int)gridDim.x + 1 : 0;

    if (warp == 16) {
        // ================= TMA producer ===================================================================
        if (lane == 0) {
            uint32_t it = 0, wit = 0;       // blocks and heads so far
            for (int k = 0; k < my_mt; ++k) {
                const MacroTile m = macro_tile(blockIdx.x + k * gridDim.x, mt_per_grid, strips, g.H, nbmax);
                const int set = m.b / g.per_set;
                for (int h = 0; h < NH; ++h, ++wit) {
                    const int wb = wit & 1, plane = m.b * NH + h;
                    ptx::mbar_wait(&wo_empty[wb], ((wit >> 1) & 1) ^ 1, status, 210);
                    ptx::mbar_expect_tx(&wo_full[wb], 8192);
                    ptx::tma_load_2d(sm + k2m::WO + wb * 8192, &map_wo, 0, (set * NH + h) * 64, &wo_full[wb]);
                    for (int b = -1; b < m.nb; ++b, ++it) {
                        const int s = it % k2m::NSTAGE;
                        uint8_t* st = sm + k2m::STG + s * k2m::STAGE_BYTES;
                        ptx::mbar_wait(&empty[s], ((it / k2m::NSTAGE) & 1) ^ 1, status, 211);
                        ptx::mbar_expect_tx(&full[s], k2m::STAGE_TX);
                        // E rows 4b+2 .. 4b+5 and V rows 4b+1 .. 4b+4 of the macro tile; plane coordinates carry the
                        // 2-cell apron (block -1 of the first macro-tile row starts V one row above the plane: rows
                        // outside the tensor read as zero and only feed values nobody uses)
                        ptx::tma_load_4d(st, &map_e, 0, m.mx0, m.my0 + 4 * b + 4, plane, &full[s]);
                        ptx::tma_load_4d(st + k2m::E_BYTES, &map_v, 0, m.mx0 + 1, m.my0 + 4 * b + 3, plane, &full[s]);
                    }
                }
            }
        }
    } else if (warp == 18) {
        // ================= TMA producer of the epilogues' state tiles ==========================================
        // Tile b of a macro tile is drained by set A (even b) or B (odd b), in this order, while the next macro tile
        // runs its first head; its state goes into that set's buffer as soon as the buffer is free.  A producer of
        // its own, so that a wait for a buffer never holds back the E / V blocks.
        if (lane == 0) {
            uint32_t nx[2] = {0, 0};        // state tiles loaded for set A and set B
            for (int k = 0; k < my_mt; ++k) {
                const MacroTile m = macro_tile(blockIdx.x + k * gridDim.x, mt_per_grid, strips, g.H, nbmax);
                for (int b = 0; b < m.nb; ++b) {
                    const int xb = b & 1;
                    ptx::mbar_wait(&x_empty[xb], (nx[xb] & 1) ^ 1, status, 212);
                    ptx::mbar_expect_tx(&x_full[xb], 16384);
                    ptx::tma_load_4d(sm + k2m::XT + xb * 16384, &map_x, 0, m.mx0, g.hx + m.my0 + b * k2m::BR, m.b, &x_full[xb]);
                    ++nx[xb];
                }
            }
        }
    } else if (warp == 17) {
        // ================= UMMA issuer ====================================================================
        if (lane == 0) {
            const uint32_t idesc = ptx::umma_idesc_bf16(128, 64);
            uint32_t v = 0, wit = 0, acc_par = 0;     // operand tiles used, heads, use parity of each accumulator
            for (int k = 0; k < my_mt; ++k) {
                const MacroTile m = macro_tile(blockIdx.x + k * gridDim.x, mt_per_grid, strips, g.H, nbmax);
                for (int h = 0; h < NH; ++h, ++wit) {
                    const int wb = wit & 1;
                    for (int b = 0; b < m.nb; ++b, ++v) {
                        const int buf = v & 1;
                        if (h == 0) ptx::mbar_wait(&acc_empty[b], ((acc_par >> b) & 1) ^ 1, status, 220);
                        if (b == 0) ptx::mbar_wait(&wo_full[wb], (wit >> 1) & 1, status, 221);
                        ptx::mbar_wait(&vp_full[buf], (v >> 1) & 1, status, 222);
                        ptx::tc_fence_after();
                        const uint64_t da = ptx::umma_desc_sw128(ptx::smem_u32(sm + k2m::A_VP + buf * 16384));
                        const uint64_t dw = ptx::umma_desc_sw128(ptx::smem_u32(sm + k2m::WO + wb * 8192));
#pragma unroll
                        for (int kk = 0; kk < 4; ++kk)
                            ptx::umma_bf16(tmem + b * 64, da + 2 * kk, dw + 2 * kk, idesc, h > 0 || kk > 0);
                        ptx::umma_commit(&vp_empty[buf]);
                        if (b == m.nb - 1) ptx::umma_commit(&wo_empty[wb]);
                        if (h == NH - 1) ptx::umma_commit(&acc_full[b]);
                    }
                }
                acc_par ^= (1u << m.nb) - 1u;
            }
        }
    } else {
        // ================= the two box-sum sets ==================================================================
        const bool is_a = warp < 8 || warp == 19;
        const int gt = warp == 19 ? 256 + lane : (is_a ? tid : tid - 256);     // thread within its set
        const int bar_ep = is_a ? 7 : 8;                        // named barrier of the set's drains (256 threads; 1-5 hand blocks over)
        float* red = reinterpret_cast<float*>(sm + k2m::RED) + (is_a ? 0 : 256);
        const int q = gt & 7, col = gt >> 3;                    // 8-dim chunk; column (A: of the 34 R columns, B: of the 32)
        uint32_t it = 0, v = 0, acc_par = 0, prev_par = 0;
        MacroTile prev;
        prev.nb = 0;
        prev.b = prev.mx0 = prev.my0 = prev.tile0 = 0;
        // the tile of macro tile `mt` in accumulator b: the epilogue, by the first 256 threads of the set
        uint32_t nxs = 0;                    // state tiles this set has drained
        uint8_t* xs = sm + k2m::XT + (is_a ? 0 : 16384);
        auto drain = [&](const MacroTile& mt, int b, uint32_t par) {
            CaTile t;
            t.b = mt.b; t.ty0 = mt.my0 + b * k2m::BR; t.tx0 = mt.mx0;
            t.index = mt.b * tiles_per_grid + mt.tile0 + b * strips;
            ptx::bar_sync(bar_ep, 256);      // the drain before this one is done with the reduction scratch
            ptx::mbar_wait(&acc_full[b], (par >> b) & 1, status, 232);
            ptx::mbar_wait(&x_full[is_a ? 0 : 1], nxs & 1, status, 233);
            ptx::tc_fence_after();
            k2_epilogue(t, tmem + b * 64, xs, scale, partial, red, bar_ep, gt, warp, g);
            if (gt == 0) {
                // X+ of the tile back to the state in one store (rows and columns past the grid are clipped); the
                // buffer goes back to the producer once the store has read it
                ptx::tma_store_4d(&map_x, xs, 0, t.tx0, g.hx + t.ty0, t.b);
                ptx::bulk_commit();
                ptx::bulk_wait_read0();
                ptx::mbar_arrive(&x_empty[is_a ? 0 : 1]);
            }
            ptx::tc_fence_before();
            ptx::mbar_arrive(&acc_empty[b]);
            ++nxs;
        };
        const int mine = is_a ? 0 : 1;       // parity of the accumulators this set drains
        V8 h2 = v8_zero(), h1 = v8_zero();   // running horizontal sums of the two rows above (of E in A, of R in B)
        uint4 ekeep0 = make_uint4(0, 0, 0, 0), ekeep1 = ekeep0;   // B: centre E of the last two rows of the block before
        const size_t vplane = (size_t)g.H * g.W * HD;
        for (int k = 0; k < my_mt; ++k) {
            const MacroTile m = macro_tile(blockIdx.x + k * gridDim.x, mt_per_grid, strips, g.H, nbmax);
            for (int h = 0; h < NH; ++h) {
                for (int b = -1; b < m.nb; ++b, ++it) {
                    const int s = it % k2m::NSTAGE;
                    uint8_t* es = sm + k2m::STG + s * k2m::STAGE_BYTES;     // [4][36] cells x 128 B
                    uint8_t* vs = es + k2m::E_BYTES;                        // [4][34] cells: V, then R in place
                    // the macro tile before: its accumulator b is drained before this one's first head overwrites it
                    if (h == 0 && b >= 0 && b < prev.nb && (b & 1) == mine && gt < 256) drain(prev, b, prev_par);
                    if (is_a) {
                        // ---- A: R = V / box3(E) for the block's four V rows, marching down ----
                        ptx::mbar_wait(&full[s], (it / k2m::NSTAGE) & 1, status, 230);
                        if (col < k2m::VW) {
#pragma unroll
                            for (int j = 0; j < k2m::BR; ++j) {
                                const uint8_t* row = es + (j * k2m::EW + col) * 128 + q * 16;
                                const uint4 e0 = *reinterpret_cast<const uint4*>(row);
                                const uint4 e1 = *reinterpret_cast<const uint4*>(row + 128);
                                const uint4 e2 = *reinterpret_cast<const uint4*>(row + 256);
                                const V8 hs = v8_sum3(e0, e1, e2);
                                if (b >= 0 || j >= 2) {      // block -1: only its last two rows have all three E rows
                                    uint4* pv = reinterpret_cast<uint4*>(vs + (j * k2m::VW + col) * 128 + q * 16);
                                    *pv = v8_pack(v8_mul(v8_unpack(*pv), v8_rcp(v8_add(v8_add(h2, h1), hs))));
                                }
                                h2 = h1; h1 = hs;
                            }
                        }
                        ptx::bar_arrive(1 + s, k2m::HANDOFF);       // R of this block is in the stage
                    } else {
                        // ---- B: V' = E * box3(R) for tile rows 4b .. 4b+3 -> A operand ----
                        const int buf = v & 1;
                        uint8_t* a_vp = sm + k2m::A_VP + buf * 16384;
                        ptx::bar_sync(1 + s, k2m::HANDOFF);
                        if (b >= 0) ptx::mbar_wait(&vp_empty[buf], ((v >> 1) & 1) ^ 1, status, 231);   // its last UMMAs are done
                        const uint8_t* ecol = es + (col + 2) * 128 + q * 16;      // this thread's column in the E rows
#pragma unroll
                        for (int j = 0; j < k2m::BR; ++j) {
                            if (b >= 0 || j >= 2) {
                                const uint8_t* row = vs + (j * k2m::VW + col) * 128 + q * 16;
                                const uint4 a0 = *reinterpret_cast<const uint4*>(row);
                                const uint4 a1 = *reinterpret_cast<const uint4*>(row + 128);
                                const uint4 a2 = *reinterpret_cast<const uint4*>(row + 256);
                                const V8 hs = v8_sum3(a0, a1, a2);
                                if (b >= 0) {
                                    // tile row j is macro-tile row 4b+j: its E came with the block before (j < 2, kept
                                    // in registers) or is row j-2 of this block's E rows
                                    const V8 e = v8_unpack(j == 0 ? ekeep0 : j == 1 ? ekeep1
                                                           : *reinterpret_cast<const uint4*>(ecol + (j - 2) * k2m::EW * 128));
                                    const uint4 out = v8_pack(v8_mul(e, v8_add(v8_add(h2, h1), hs)));
                                    *reinterpret_cast<uint4*>(a_vp + swz(j * k2m::SW + col, q)) = out;
                                    const int orow = m.my0 + 4 * b + j, ocol = m.mx0 + col;
                                    if (vprime != nullptr && orow < g.H && ocol < g.W)
                                        *reinterpret_cast<uint4*>(vprime + ((size_t)m.b * NH + h) * vplane +
                                                                  ((size_t)orow * g.W + ocol) * HD + q * 8) = out;
                                }
                                h2 = h1; h1 = hs;
                            }
                        }
                        ekeep0 = *reinterpret_cast<const uint4*>(ecol + 2 * k2m::EW * 128);
                        ekeep1 = *reinterpret_cast<const uint4*>(ecol + 3 * k2m::EW * 128);
                        if (b >= 0) {
                            ptx::fence_proxy_async();
                            ptx::mbar_arrive(&vp_full[buf]);
                            ++v;
                        }
                        ptx::mbar_arrive(&empty[s]);
                    }
                }
                // accumulators of the macro tile before that this one does not reach (it has fewer blocks)
                if (h == 0 && gt < 256)
                    for (int b = m.nb; b < prev.nb; ++b)
                        if ((b & 1) == mine) drain(prev, b, prev_par);
            }
            prev = m;
            prev_par = acc_par;
            acc_par ^= (1u << m.nb) - 1u;
        }
        if (gt < 256)
            for (int b = 0; b < prev.nb; ++b)
                if ((b & 1) == mine) drain(prev, b, prev_par);
        if (gt == 0) ptx::bulk_wait0();      // this set's stores of X+ are complete
    }
    ptx::tc_fence_before();
    __syncthreads();
    if (warp == 0) ptx::tmem_dealloc(tmem, k2m::TMEM_COLS);
}

// =============================================================================================================
// host side
inline const char*& bf16_error_ref() { static const char* e = ""; return e; }
inline const char* bf16_error() { return bf16_error_ref(); }

inline void bf16_plan(Bf16Plan& p, const Geom& g) {
    p.tiles_x = (g.W + TBW - 1) / TBW;
    p.k1_tiles = p.tiles_x * ((g.H + 2 * g.he + TBH - 1) / TBH);
    p.strips = (g.W + k2m::SW - 1) / k2m::SW;
    p.k2_tiles = p.strips * ((g.H + k2m::BR - 1) / k2m::BR);      // one partial per 4 x 32 tile
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
                      const __nv_bfloat16* V, const __nv_bfloat16* X, const Geom& g, int num_sms) {
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
    if (make_plane_map(enc, &p.map_e, E, g, k2m::EW, k2m::BR) || make_plane_map(enc, &p.map_v, V, g, k2m::VW, k2m::BR) ||
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
    {
        // the state as k2's epilogue sees it: the rows below the own rows (a stripe's bottom halo) are left out of
        // the tensor, so a store of a tile that hangs over the last own row is clipped there
        const cuuint64_t dims[4] = {64, (cuuint64_t)g.W, (cuuint64_t)(g.hx + g.H), (cuuint64_t)g.B};
        const cuuint64_t strides[3] = {128, (cuuint64_t)g.W * 128, (cuuint64_t)g.state_rows() * g.W * 128};
        const cuuint32_t box[4] = {64, k2m::SW, k2m::BR, 1};
        const cuuint32_t estr[4] = {1, 1, 1, 1};
        if (enc(&p.map_x, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 4, const_cast<__nv_bfloat16*>(X), dims, strides, box, estr,
                CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B,
                CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE) != CUDA_SUCCESS) {
            bf16_error_ref() = "cuTensorMapEncodeTiled rejected the state layout";
            return -1;
        }
    }
    p.k1_aligned = g.W % TBW == 0 && (!g.wrap_y || g.H % TBH == 0);
    if (cudaFuncSetAttribute(k1_bf16<true>, cudaFuncAttributeMaxDynamicSharedMemorySize, k1b::SMEM) != cudaSuccess ||
        cudaFuncSetAttribute(k1_bf16<false>, cudaFuncAttributeMaxDynamicSharedMemorySize, k1b::SMEM) != cudaSuccess ||
        cudaFuncSetAttribute(k2_bf16, cudaFuncAttributeMaxDynamicSharedMemorySize, k2m::SMEM) != cudaSuccess) {
        bf16_error_ref() = "could not opt in to the kernels' dynamic shared memory";
        return -1;
    }
    const long long total1 = (long long)p.k1_tiles * g.B;
    p.k1_grid = (int)(total1 < num_sms ? total1 : num_sms);
    // k2: blocks per macro tile.  A taller macro tile re-primes its march less often (nb + 1 blocks of work for nb
    // tiles) but gives fewer, coarser units to spread over the SMs: take the height with the best product of the two.
    long long total_mt = 0;
    double best = -1.0;
    const int rows4 = (g.H + k2m::BR - 1) / k2m::BR;
    for (int nb = k2m::NB; nb >= 1; nb >>= 1) {
        const int mt_rows = (rows4 + nb - 1) / nb;
        const long long total = (long long)p.strips * mt_rows * g.B;
        const double per_mt = (double)rows4 / mt_rows;                         // tiles per macro tile on average
        const long long waves = (total + num_sms - 1) / num_sms;
        const double eff = per_mt / (per_mt + 1.0) * (double)total / (double)(waves * num_sms);
        if (eff > best) { best = eff; p.nbmax = nb; p.mt_per_grid = p.strips * mt_rows; total_mt = total; }
    }
    p.k2_grid = (int)(total_mt < num_sms ? total_mt : num_sms);
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
    k2_bf16<<<p.k2_grid, k2m::THREADS, k2m::SMEM, st>>>(p.map_wo, p.map_e, p.map_v, p.map_x, scale, partial, vprime, status,
                                                        p.mt_per_grid * g.B, p.mt_per_grid, p.strips, p.k2_tiles, p.nbmax, g);
    return cudaGetLastError() == cudaSuccess ? 0 : -1;
}

}  // namespace slime
