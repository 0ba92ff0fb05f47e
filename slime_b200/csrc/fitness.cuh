// Fitness reduction: per (grid, head) 64x64 Gram of the redistributed value V', Jacobi eigenvalues,
// exp-entropy rank, Pearson coherence between the last two steps, fitness = rank x coherence.
// Replaces gpu_svd_kernel / effective_rank_kernel / coherence_kernel / fitness_fused_kernel
// (slime/kernels/warp_ca.cu:66-226).  Gram and Jacobi run in fp64: the small eigenvalues carry most of the
// entropy's sensitivity, and an fp32 Gram loses them.
#pragma once
#include "ca_aux.cuh"
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

// One 128-thread block per (grid, head): sum the Gram partials, diagonalise by two-sided Jacobi with a
// round-robin (tournament) ordering - 32 disjoint rotations per round, 63 rounds per sweep - until the
// off-diagonal Frobenius norm is <= 1e-6 x the matrix norm, plus one more sweep, at most 30 sweeps
// (rotation formula of slime/kernels/warp_ca.cu:51-63, sweep limit :20), then the exp-entropy rank
// p = l/(sum l + 1e-7), rank = exp(-sum p ln(p + 1e-7))  (slime/kernels/warp_ca.cu:107-144).
// Thread t works on rotation pair t % 32 and on a quarter (t / 32) of the 64 elements of its two columns / rows.
constexpr int JACOBI_THREADS = 128;
__device__ __forceinline__ double jacobi_block_sum(double v, double* red) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    __syncthreads();
    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = v;
    __syncthreads();
    return (red[0] + red[1]) + (red[2] + red[3]);
}
__global__ void __launch_bounds__(JACOBI_THREADS)
k_jacobi_rank(const double* __restrict__ gram_part, int splits, float* __restrict__ head_rank) {
    __shared__ double A[64 * JSTRIDE];
    __shared__ double red[4];
    const int m = blockIdx.x, tid = threadIdx.x, pair = tid & 31, k0 = (tid >> 5) * 16;
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
            int p, q;
            if (pair == 0) { p = 63; q = round; }
            else { p = (round + pair) % 63; q = (round + 63 - pair) % 63; }
            if (p > q) { const int t = p; p = q; q = t; }
            const double apq = A[p * JSTRIDE + q];
            double c = 1.0, s = 0.0;
            if (apq != 0.0) {
                const double tau = (A[q * JSTRIDE + q] - A[p * JSTRIDE + p]) / (2.0 * apq);
                const double t = (tau >= 0.0 ? 1.0 : -1.0) / (fabs(tau) + sqrt(1.0 + tau * tau));
                c = 1.0 / sqrt(1.0 + t * t);
                s = t * c;
            }
            __syncthreads();
            for (int k = k0; k < k0 + 16; ++k) {    // columns p, q
                const double akp = A[k * JSTRIDE + p], akq = A[k * JSTRIDE + q];
                A[k * JSTRIDE + p] = c * akp - s * akq;
                A[k * JSTRIDE + q] = s * akp + c * akq;
            }
            __syncthreads();
            for (int k = k0; k < k0 + 16; ++k) {    // rows p, q
                const double apk = A[p * JSTRIDE + k], aqk = A[q * JSTRIDE + k];
                A[p * JSTRIDE + k] = c * apk - s * aqk;
                A[q * JSTRIDE + k] = s * apk + c * aqk;
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
// part[(b*splits + split)][5] = {sum a, sum b, sum aa, sum bb, sum ab}.
template <typename T>
__global__ void __launch_bounds__(256)
k_pearson(const T* __restrict__ va, const T* __restrict__ vb, size_t per_grid, double* __restrict__ part) {
    __shared__ double red[5][256];
    const int split = blockIdx.x, b = blockIdx.y, splits = gridDim.x;
    const size_t chunk = (per_grid + splits - 1) / splits;
    const size_t lo = (size_t)split * chunk;
    const size_t hi = lo + chunk < per_grid ? lo + chunk : per_grid;
    const T* a = va + (size_t)b * per_grid;
    const T* c = vb + (size_t)b * per_grid;
    double s[5] = {0, 0, 0, 0, 0};
    for (size_t i = lo + threadIdx.x; i < hi; i += 256) {
        const double x = to_f32<T>(a[i]), y = to_f32<T>(c[i]);
        s[0] += x; s[1] += y; s[2] = fma(x, x, s[2]); s[3] = fma(y, y, s[3]); s[4] = fma(x, y, s[4]);
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
