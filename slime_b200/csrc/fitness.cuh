// Fitness reduction: per (grid, head) 64x64 Gram of the redistributed value V', Jacobi eigenvalues,
// exp-entropy rank, Pearson coherence between the last two steps, fitness = rank x coherence.
// Replaces gpu_svd_kernel / effective_rank_kernel / coherence_kernel / fitness_fused_kernel
// (slime/kernels/warp_ca.cu:66-226).  Gram and Jacobi run in fp64: the small eigenvalues carry most of the
// entropy's sensitivity, and an fp32 Gram loses them.
#pragma once
#include "ca_aux.cuh"
#include "ca_bf16.cuh"
#include "common.cuh"

namespace slime {

constexpr int GRAM_CHUNK = 2048;   // cells per Gram partial
constexpr int JSTRIDE = 65;        // padded row stride of the Jacobi matrix in shared memory (doubles)

// gram_part[((b*8+h)*splits + split)][64][64] (fp64) over cells [split*GRAM_CHUNK, ...) of plane (b,h).
// The Gram matrix is symmetric: only the 136 4x4 blocks on or above the diagonal are accumulated (one thread
// each, 160 threads per block) and each is written to both places.  A chunk of 64 cells is converted to fp64
// once, on its way into shared memory (the conversion is the slow instruction here: converting at the point of
// use cost one conversion per two multiply-adds and made them the bottleneck).  Each 4-value block of a cell is
// kept as two 16-byte halves in two planes, so a warp's loads of consecutive blocks are consecutive 16-byte
// words: no bank conflicts.
constexpr int GRAM_THREADS = 160;
template <typename T>
__global__ void __launch_bounds__(GRAM_THREADS, 6)
k_gram(const T* __restrict__ vp, int cells, double* __restrict__ gram_part) {
    __shared__ __align__(16) double2 flo[64][16];      // values 4 blk + 0, 4 blk + 1 of cell s
    __shared__ __align__(16) double2 fhi[64][16];      // values 4 blk + 2, 4 blk + 3
    const int split = blockIdx.x, h = blockIdx.y, b = blockIdx.z, splits = gridDim.x;
    const T* plane = vp + ((size_t)b * NH + h) * (size_t)cells * HD;
    // thread t -> block (bi, bj), bi <= bj, rows of the upper triangle laid end to end: row bi starts at
    // bi * 16 - bi * (bi - 1) / 2
    int bi = 0, rest = threadIdx.x;
    const bool live = threadIdx.x < 136;
    if (live) { while (rest >= 16 - bi) { rest -= 16 - bi; ++bi; } } else rest = 0;
    const int bj = bi + rest, ti = bi * 4, tj = bj * 4;
    double acc[4][4];
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) acc[i][j] = 0.0;
    const int lo = split * GRAM_CHUNK;
    const int hi = min(lo + GRAM_CHUNK, cells);
    for (int s0 = lo; s0 < hi; s0 += 64) {
        __syncthreads();
        for (int i = threadIdx.x; i < 64 * 32; i += GRAM_THREADS) {       // one pair of adjacent values per step
            const int sl = i >> 5, pr = i & 31, s = s0 + sl;
            double2 v = make_double2(0.0, 0.0);
            if (s < hi) {
                v.x = (double)to_f32<T>(plane[(size_t)s * HD + 2 * pr]);
                v.y = (double)to_f32<T>(plane[(size_t)s * HD + 2 * pr + 1]);
            }
            if (pr & 1) fhi[sl][pr >> 1] = v; else flo[sl][pr >> 1] = v;
        }
        __syncthreads();
        if (live) {
#pragma unroll 8
            for (int s = 0; s < 64; ++s) {
                const double2 a0 = flo[s][bi], a1 = fhi[s][bi], c0 = flo[s][bj], c1 = fhi[s][bj];
                const double av[4] = {a0.x, a0.y, a1.x, a1.y};
                const double cv[4] = {c0.x, c0.y, c1.x, c1.y};
#pragma unroll
                for (int i = 0; i < 4; ++i)
#pragma unroll
                    for (int j = 0; j < 4; ++j) acc[i][j] = fma(av[i], cv[j], acc[i][j]);
            }
        }
    }
    if (!live) return;
    double* out = gram_part + (((size_t)b * NH + h) * splits + split) * (HD * HD);
#pragma unroll
    for (int i = 0; i < 4; ++i)
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            out[(ti + i) * HD + tj + j] = acc[i][j];
            if (ti != tj) out[(tj + j) * HD + ti + i] = acc[i][j];
        }
}

// The same Gram partials for bf16 planes on the tensor cores.  One CTA per (grid, head) plane walks the plane in tiles
// of 128 cells; a tile [128 cells][64 dims] lands in shared memory by TMA with the 128-byte swizzle, which is exactly
// the MN-major operand layout of tcgen05 (one 128-byte row of the 64 dims per cell), so the one tile is both operands of
// D[64 x 64] += F^T F: eight tcgen05.mma of M = 64, N = 64, K = 16 cells, fp32 accumulation in 64 TMEM columns (the
// products of bf16 values are exact in fp32).  After every GRAM_CHUNK cells the accumulator is written out as one fp64
// partial - the same [plane][split][64][64] layout the SIMT kernel fills - and cleared by the next chunk's first
// instruction, so chunks are still summed in fp64 by k_jacobi_rank.  An M = 64 accumulator keeps row r in TMEM lane
// 32 * (r / 16) + r % 16: warp w's first sixteen lanes hold rows 16 w .. 16 w + 15.
namespace gtc {
constexpr int TILE = 128, STAGES = 4, TILE_BYTES = TILE * 128;
constexpr int BARS = STAGES * TILE_BYTES, TMEM_PTR = BARS + (2 * STAGES + 2) * 8, BYTES = TMEM_PTR + 16, SMEM = BYTES + 1024;
constexpr uint32_t IDESC = ptx::umma_idesc_bf16(64, 64) | (1u << 15) | (1u << 16);     // both operands MN-major
}  // namespace gtc
__global__ void __launch_bounds__(128)
k_gram_tc(const __grid_constant__ CUtensorMap map_vp, int cells, int splits, double* __restrict__ gram_part,
          int* __restrict__ status) {
    extern __shared__ uint8_t smem_raw[];
    uint8_t* sm = align1024(smem_raw);
    uint64_t* full = reinterpret_cast<uint64_t*>(sm + gtc::BARS);     // [4] tile landed            (waits: UMMA issuer)
    uint64_t* empty = full + gtc::STAGES;                             // [4] its UMMAs are done     (waits: TMA producer)
    uint64_t* acc_full = empty + gtc::STAGES;                         //     chunk accumulated      (waits: all)
    uint64_t* acc_empty = acc_full + 1;                               //     chunk written out      (waits: UMMA issuer)
    uint32_t* tmem_ptr = reinterpret_cast<uint32_t*>(sm + gtc::TMEM_PTR);
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31, plane = blockIdx.x;
    if (tid == 0) {
        for (int i = 0; i < gtc::STAGES; ++i) { ptx::mbar_init(&full[i], 1); ptx::mbar_init(&empty[i], 1); }
        ptx::mbar_init(acc_full, 1);
        ptx::mbar_init(acc_empty, 128);
        ptx::fence_barrier_init();
        ptx::prefetch_tmap(&map_vp);
    }
    if (warp == 0) ptx::tmem_alloc(tmem_ptr, 64);
    ptx::tc_fence_before();
    __syncthreads();
    ptx::tc_fence_after();
    const uint32_t tmem = *tmem_ptr;
    uint32_t it = 0;       // tiles so far (the producer and the issuer count the same way)
    for (int split = 0; split < splits; ++split) {
        const int lo = split * GRAM_CHUNK, hi = min(lo + GRAM_CHUNK, cells);
        const int n_tiles = (hi - lo + gtc::TILE - 1) / gtc::TILE;
        if (warp == 0 && lane == 0) {
            for (int t = 0; t < n_tiles; ++t) {
                const uint32_t i = it + t, s = i % gtc::STAGES;
                ptx::mbar_wait(&empty[s], ((i / gtc::STAGES) & 1) ^ 1, status, 410);
                ptx::mbar_expect_tx(&full[s], gtc::TILE_BYTES);
                // cells past the end of the plane read as zero and add nothing (the last chunk ends at the plane's end:
                // a tile never reaches into the next chunk)
                ptx::tma_load_3d(sm + s * gtc::TILE_BYTES, &map_vp, 0, lo + t * gtc::TILE, plane, &full[s]);
            }
        } else if (warp == 1 && lane == 0) {
            ptx::mbar_wait(acc_empty, (split & 1) ^ 1, status, 411);
            ptx::tc_fence_after();
            for (int t = 0; t < n_tiles; ++t) {
                const uint32_t i = it + t, s = i % gtc::STAGES;
                ptx::mbar_wait(&full[s], (i / gtc::STAGES) & 1, status, 412);
                ptx::tc_fence_after();
                const uint64_t d = ptx::umma_desc_sw128(ptx::smem_u32(sm + s * gtc::TILE_BYTES));
#pragma unroll
                for (int ks = 0; ks < 8; ++ks)      // 16 cells per step: 2048 bytes = 128 sixteen-byte units further
                    ptx::umma_bf16(tmem, d + 128 * ks, d + 128 * ks, gtc::IDESC, t > 0 || ks > 0);
                ptx::umma_commit(&empty[s]);
            }
            ptx::umma_commit(acc_full);
        }
        it += n_tiles;
        __syncwarp();
        ptx::mbar_wait(acc_full, split & 1, status, 413);
        ptx::tc_fence_after();
        double* out = gram_part + ((size_t)plane * splits + split) * (HD * HD) + (size_t)(warp * 16 + (lane & 15)) * HD;
#pragma unroll
        for (int c = 0; c < HD; c += 16) {
            uint32_t r[16];
            ptx::tmem_ld16(tmem + ((uint32_t)(warp * 32) << 16) + c, r);
            ptx::tmem_ld_wait();
            if (lane < 16) {
#pragma unroll
                for (int k = 0; k < 16; k += 2)
                    *reinterpret_cast<double2*>(out + c + k) = make_double2((double)__uint_as_float(r[k]), (double)__uint_as_float(r[k + 1]));
            }
        }
        ptx::tc_fence_before();
        ptx::mbar_arrive(acc_empty);
    }
    ptx::tc_fence_before();
    __syncthreads();
    if (warp == 0) ptx::tmem_dealloc(tmem, 64);
}

// Tensor map over a V' buffer [planes][cells][64] bf16 for k_gram_tc: box 64 dims x 128 cells x 1 plane, 128B swizzle.
inline int gram_tc_map(CUtensorMap* map, const void* vp, int planes, int cells) {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) != cudaSuccess || !fn ||
        q != cudaDriverEntryPointSuccess)
        return -1;
    const cuuint64_t dims[3] = {64, (cuuint64_t)cells, (cuuint64_t)planes};
    const cuuint64_t strides[2] = {128, (cuuint64_t)cells * 128};
    const cuuint32_t box[3] = {64, gtc::TILE, 1};
    const cuuint32_t estr[3] = {1, 1, 1};
    const CUresult r = reinterpret_cast<EncodeTiledFn>(fn)(map, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(vp), dims,
                                                         strides, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                                         CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) return -1;
    return cudaFuncSetAttribute(k_gram_tc, cudaFuncAttributeMaxDynamicSharedMemorySize, gtc::SMEM) == cudaSuccess ? 0 : -1;
}

// One 256-thread block per (grid, head): sum the Gram partials, diagonalise by two-sided Jacobi with a
// round-robin (tournament) ordering - 32 disjoint rotations per round, applied as 1024 independent 2 x 2 blocks, 63
// rounds per sweep - until the
// off-diagonal Frobenius norm is <= 1e-6 x the matrix norm, plus one more sweep, at most 30 sweeps
// (rotation formula of slime/kernels/warp_ca.cu:51-63, sweep limit :20), then the exp-entropy rank
// p = l/(sum l + 1e-7), rank = exp(-sum p ln(p + 1e-7))  (slime/kernels/warp_ca.cu:107-144).
constexpr int JACOBI_THREADS = 256;
// pair `i` of round `r` of the 64-player round-robin tournament: 32 disjoint index pairs per round, 63 rounds
__device__ __forceinline__ void jacobi_pair(int r, int i, int& p, int& q) {
    if (i == 0) { p = 63; q = r; }
    else { p = (r + i) % 63; q = (r + 63 - i) % 63; }
}
__device__ __forceinline__ double jacobi_block_sum(double v, double* red) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    return ((red[0] + red[1]) + (red[2] + red[3])) + ((red[4] + red[5]) + (red[6] + red[7]));
}
__global__ void __launch_bounds__(JACOBI_THREADS)
k_jacobi_rank(const double* __restrict__ gram_part, int splits, float* __restrict__ head_rank) {
    __shared__ double A[64 * JSTRIDE];
    __shared__ double red[8];
    __shared__ double2 cs[32];          // (cos, sin) of the round's 32 rotations
    const int m = blockIdx.x, tid = threadIdx.x;
    const double* src = gram_part + (size_t)m * splits * (HD * HD);
    double fro2 = 0.0;
    for (int i = tid; i < HD * HD; i += JACOBI_THREADS) {
        double s = 0.0;
        for (int k = 0; k < splits; ++k) s += src[(size_t)k * (HD * HD) + i];
        A[(i >> 6) * JSTRIDE + (i & 63)] = s;
        fro2 += s * s;
    }
    fro2 = jacobi_block_sum(fro2, red);

    int extra = 0;
    for (int sweep = 0; sweep < 30; ++sweep) {
        double off2 = 0.0;
        for (int i = tid; i < HD * HD; i += JACOBI_THREADS) {
            const int r = i >> 6, c = i & 63;
            if (r != c) { const double v = A[r * JSTRIDE + c]; off2 += v * v; }
        }
        off2 = jacobi_block_sum(off2, red);          // the same value in every thread: the exit below is uniform
        if (off2 <= 1e-12 * fro2) { if (extra) break; extra = 1; }
        for (int round = 0; round < 63; ++round) {
            // (p, q) of a pair is used as the tournament hands it out, not ordered: a warp's values of p, and of q, are
            // then consecutive indices (mod 63), which land in distinct banks; the matrix keeps both triangles, so
            // A[p][q] is there whichever of the two is larger, and the rotation zeroes it either way
            if (tid < 32) {
                int p, q;
                jacobi_pair(round, tid, p, q);
                const double apq = A[p * JSTRIDE + q];
                double c = 1.0, sn = 0.0;
                if (apq != 0.0) {
                    // The tangent of the rotation angle only decides how much of A[p][q] the rotation removes (all of
                    // it, to fp32 accuracy here: three fp64 divisions and square roots on one warp were the longest
                    // serial stretch of a round); what has to be exact is that the rotation is orthogonal, and
                    // c = 1 / sqrt(1 + t^2), s = t c in fp64 make it so for whatever t.
                    const float tau = (float)(A[q * JSTRIDE + q] - A[p * JSTRIDE + p]) / (2.f * (float)apq);
                    const float tf = (tau >= 0.f ? 1.f : -1.f) / (fabsf(tau) + sqrtf(1.f + tau * tau));
                    const double t = isfinite(tf) ? (double)tf : 0.0;
                    c = rsqrt(1.0 + t * t);
                    sn = t * c;
                }
                cs[tid] = make_double2(c, sn);
            }
            __syncthreads();
            // The round's 32 rotations touch disjoint index pairs, so A'' = J^T A J falls apart into 32 x 32 independent
            // 2 x 2 blocks: rows (p, q) of one pair against columns (p', q') of another.  A thread takes 4 blocks:
            // columns first, then rows, exactly the arithmetic of rotating all columns and then all rows, but every
            // element is read and written once per round instead of twice, with one barrier fewer.
            {
                int p, q;
                // a warp holds the 32 row pairs of one column pair: its 8-byte accesses go to (almost) consecutive rows
                // of one column, i.e. distinct banks (the row stride is odd)
                jacobi_pair(round, tid & 31, p, q);
                const double2 rc = cs[tid & 31];
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const int cp = (tid >> 5) * 4 + j;
                    int p2, q2;
                    jacobi_pair(round, cp, p2, q2);
                    const double2 cc = cs[cp];
                    const double a_pp = A[p * JSTRIDE + p2], a_pq = A[p * JSTRIDE + q2];
                    const double a_qp = A[q * JSTRIDE + p2], a_qq = A[q * JSTRIDE + q2];
                    const double b_pp = cc.x * a_pp - cc.y * a_pq, b_pq = cc.y * a_pp + cc.x * a_pq;      // columns p', q'
                    const double b_qp = cc.x * a_qp - cc.y * a_qq, b_qq = cc.y * a_qp + cc.x * a_qq;
                    A[p * JSTRIDE + p2] = rc.x * b_pp - rc.y * b_qp;                                        // rows p, q
                    A[p * JSTRIDE + q2] = rc.x * b_pq - rc.y * b_qq;
                    A[q * JSTRIDE + p2] = rc.y * b_pp + rc.x * b_qp;
                    A[q * JSTRIDE + q2] = rc.y * b_pq + rc.x * b_qq;
                }
            }
            __syncthreads();
        }
    }
    if (tid >= 32) return;
    const int lane = tid;
    double l0 = fmax(A[lane * JSTRIDE + lane], 0.0), l1 = fmax(A[(lane + 32) * JSTRIDE + lane + 32], 0.0);
    double sum = l0 + l1;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
    const double p0 = l0 / (sum + 1e-7), p1 = l1 / (sum + 1e-7);
    double ent = -(p0 * log(p0 + 1e-7) + p1 * log(p1 + 1e-7));
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) ent += __shfl_xor_sync(0xffffffffu, ent, o);
    if (lane == 0) head_rank[m] = (float)exp(ent);
}

// Raw moments of (a, b) = (V' of step n-1, V' of step n) for one grid, fp64:
// part[(b*splits + split)][5] = {sum a, sum b, sum aa, sum bb, sum ab}.  Sixteen bytes per load (4 fp32 or 8 bf16
// values); per_grid is a multiple of 512.
template <typename T> struct PearsonVec;
template <> struct PearsonVec<float> {
    static constexpr int N = 4;
    static __device__ __forceinline__ void load(const float* p, float (&f)[8]) {
        const float4 v = *reinterpret_cast<const float4*>(p);
        f[0] = v.x; f[1] = v.y; f[2] = v.z; f[3] = v.w;
    }
};
template <> struct PearsonVec<__nv_bfloat16> {
    static constexpr int N = 8;
    static __device__ __forceinline__ void load(const __nv_bfloat16* p, float (&f)[8]) { unpack8(*reinterpret_cast<const uint4*>(p), f); }
};
template <typename T>
__global__ void __launch_bounds__(256)
k_pearson(const T* __restrict__ va, const T* __restrict__ vb, size_t per_grid, double* __restrict__ part) {
    __shared__ double red[5][256];
    constexpr int N = PearsonVec<T>::N;
    const int split = blockIdx.x, b = blockIdx.y, splits = gridDim.x;
    const size_t vecs = per_grid / N;
    const size_t chunk = (vecs + splits - 1) / splits;
    const size_t lo = (size_t)split * chunk;
    const size_t hi = lo + chunk < vecs ? lo + chunk : vecs;
    const T* a = va + (size_t)b * per_grid;
    const T* c = vb + (size_t)b * per_grid;
    double s[5] = {0, 0, 0, 0, 0};
    for (size_t i = lo + threadIdx.x; i < hi; i += 256) {
        float x[8], y[8];
        PearsonVec<T>::load(a + i * N, x);
        PearsonVec<T>::load(c + i * N, y);
#pragma unroll
        for (int k = 0; k < N; ++k) {
            const double xd = x[k], yd = y[k];
            s[0] += xd; s[1] += yd; s[2] = fma(xd, xd, s[2]); s[3] = fma(yd, yd, s[3]); s[4] = fma(xd, yd, s[4]);
        }
    }
    for (int k = 0; k < 5; ++k) red[k][threadIdx.x] = s[k];
    __syncthreads();
    for (int w = 128; w > 0; w >>= 1) {
        if (threadIdx.x < w)
            for (int k = 0; k < 5; ++k) red[k][threadIdx.x] += red[k][threadIdx.x + w];
        __syncthreads();
    }
    if (threadIdx.x < 5) part[((size_t)b * splits + split) * 5 + threadIdx.x] = red[threadIdx.x][0];
}

// out[b] = {rank, coherence, fitness, hunger}: fitness = rank x coherence (slime/kernels/warp_ca.cu:219),
// hunger = 1 - coherence (slime/kernels/warp_ca.cu:238).
__global__ void k_fitness_final(const float* __restrict__ head_rank, const double* __restrict__ part, int splits,
                                double n, float* __restrict__ out, int B) {
    const int b = blockIdx.x * blockDim.x + threadIdx.x;
    if (b >= B) return;
    double s[5] = {0, 0, 0, 0, 0};
    for (int k = 0; k < splits; ++k)
        for (int j = 0; j < 5; ++j) s[j] += part[((size_t)b * splits + k) * 5 + j];
    const double cov = s[4] - s[0] * s[1] / n;
    const double va = s[2] - s[0] * s[0] / n, vb = s[3] - s[1] * s[1] / n;
    const double coh = cov / sqrt(va * vb);
    double rk = 0.0;
    for (int h = 0; h < NH; ++h) rk += (double)head_rank[b * NH + h];
    rk /= NH;
    out[b * 4 + 0] = (float)rk;
    out[b * 4 + 1] = (float)coh;
    out[b * 4 + 2] = (float)(rk * coh);
    out[b * 4 + 3] = (float)(1.0 - coh);
}

}  // namespace slime
