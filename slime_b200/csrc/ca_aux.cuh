// Small kernels around the step: deterministic per-channel sums, the lazy renormalisation scale,
// dtype conversion on the way in and out, the 1-channel lift and the pooled readout.
#pragma once
#include "common.cuh"

namespace slime {

template <typename T> __device__ __forceinline__ float to_f32(T v);
template <> __device__ __forceinline__ float to_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ float to_f32<__nv_bfloat16>(__nv_bfloat16 v) { return __bfloat162float(v); }
template <typename T> __device__ __forceinline__ T from_f32(float v);
template <> __device__ __forceinline__ float from_f32<float>(float v) { return v; }
template <> __device__ __forceinline__ __nv_bfloat16 from_f32<__nv_bfloat16>(float v) { return __float2bfloat16_rn(v); }

// Per-channel sums of the own rows of the stored state, one partial per 256-cell chunk:
// partial[b][chunk][c] (fp32 over 64 cells per thread, combined in a fixed order).
template <typename T>
__global__ void __launch_bounds__(256)
k_channel_partials(const T* __restrict__ X, float* __restrict__ partial, Geom g) {
    __shared__ float red[4][64];
    const int b = blockIdx.y, c = threadIdx.x & 63, sub = threadIdx.x >> 6;
    const size_t cells = (size_t)g.H * g.W;
    const size_t first = (size_t)blockIdx.x * 256 + sub * 64;
    const T* base = X + ((size_t)b * g.state_rows() + g.hx) * g.W * NC;
    float s = 0.f;
    for (int i = 0; i < 64; ++i) {
        const size_t cell = first + i;
        if (cell < cells) s += to_f32<T>(base[cell * NC + c]);
    }
    red[sub][c] = s;
    __syncthreads();
    if (sub == 0) partial[((size_t)b * gridDim.x + blockIdx.x) * NC + c] = (red[0][c] + red[1][c]) + (red[2][c] + red[3][c]);
}

// Stage 1 of the cross-tile reduction: segment s of grid b sums its share of the partials in fp64.  lo_offset != 0:
// every partial is a float pair, the remainder lo_offset floats after the value (the fp32 step kernel's tile sums).
__global__ void __launch_bounds__(256)
k_reduce_partials(const float* __restrict__ partial, int n_partials, double* __restrict__ seg_sums, size_t lo_offset = 0) {
    __shared__ double red[4][64];
    const int b = blockIdx.y, c = threadIdx.x & 63, sub = threadIdx.x >> 6;
    const int nseg = gridDim.x;
    const int per_seg = (n_partials + nseg - 1) / nseg;
    const int per_sub = (per_seg + 3) / 4;
    const int lo = blockIdx.x * per_seg + sub * per_sub;
    int hi = lo + per_sub;
    const int seg_hi = min((blockIdx.x + 1) * per_seg, n_partials);
    if (hi > seg_hi) hi = seg_hi;
    double s = 0.0;
    for (int t = lo; t < hi; ++t) {
        const size_t o = ((size_t)b * n_partials + t) * NC + c;
        s += (double)partial[o];
        if (lo_offset) s += (double)partial[o + lo_offset];
    }
    red[sub][c] = s;
    __syncthreads();
    if (sub == 0) seg_sums[((size_t)b * nseg + blockIdx.x) * NC + c] = (red[0][c] + red[1][c]) + (red[2][c] + red[3][c]);
}

// Both stages of the cross-tile reduction in one launch: segment s of grid b sums its share of the partials in fp64
// (as k_reduce_partials), and the block that finishes last for its grid (a ticket per grid, handed back at zero) adds
// the segments in their fixed order, so the result does not depend on which block that is.
// mode 0: sums only; 1: also mass = sums and scale = 1 (a freshly loaded state); 2: also scale = mass / sums.
__global__ void __launch_bounds__(256)
k_reduce_finish(const float* __restrict__ partial, int n_partials, double* __restrict__ seg_sums, size_t lo_offset,
                int* __restrict__ tickets, double* __restrict__ sums, double* __restrict__ mass,
                float* __restrict__ scale, int mode) {
    __shared__ double red[4][64];
    __shared__ int is_last;
    const int b = blockIdx.y, c = threadIdx.x & 63, sub = threadIdx.x >> 6;
    const int nseg = gridDim.x;
    const int per_seg = (n_partials + nseg - 1) / nseg;
    const int per_sub = (per_seg + 3) / 4;
    const int lo = blockIdx.x * per_seg + sub * per_sub;
    int hi = lo + per_sub;
    const int seg_hi = min((blockIdx.x + 1) * per_seg, n_partials);
    if (hi > seg_hi) hi = seg_hi;
    double s = 0.0;
    for (int t = lo; t < hi; ++t) {
        const size_t o = ((size_t)b * n_partials + t) * NC + c;
        s += (double)partial[o];
        if (lo_offset) s += (double)partial[o + lo_offset];
    }
    red[sub][c] = s;
    __syncthreads();
    if (sub == 0) {
        seg_sums[((size_t)b * nseg + blockIdx.x) * NC + c] = (red[0][c] + red[1][c]) + (red[2][c] + red[3][c]);
        __threadfence();
    }
    __syncthreads();
    if (threadIdx.x == 0) is_last = atomicAdd(&tickets[b], 1) == nseg - 1;
    __syncthreads();
    if (!is_last) return;
    __threadfence();
    if (sub == 0) {
        double t = 0.0;
        for (int i = 0; i < nseg; ++i) t += __ldcg(&seg_sums[((size_t)b * nseg + i) * NC + c]);
        sums[b * NC + c] = t;
        if (mode == 1) { mass[b * NC + c] = t; scale[b * NC + c] = 1.f; }
        if (mode == 2) scale[b * NC + c] = (float)(mass[b * NC + c] / t);
    }
    if (threadIdx.x == 0) tickets[b] = 0;
}

// scale = mass / sums from buffers the caller may have all-reduced.
__global__ void k_scale_from_sums(const double* __restrict__ sums, const double* __restrict__ mass,
                                  float* __restrict__ scale, int n) {
    const int i = blockIdx.x * blockDim.x + threadIdx.x;
    if (i < n) scale[i] = (float)(mass[i] / sums[i]);
}

// dense [B][H][W][64] (TI) -> own rows of the state buffer (TO); halo rows untouched.
template <typename TI, typename TO>
__global__ void k_state_in(const TI* __restrict__ src, TO* __restrict__ X, Geom g) {
    const size_t per = (size_t)g.H * g.W * NC;
    const size_t n = per * g.B;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        const size_t b = i / per, o = i % per;
        X[(b * g.state_rows() + g.hx) * g.W * NC + o] = from_f32<TO>(to_f32<TI>(src[i]));
    }
}

// own rows of the state buffer times the pending scale -> dense [B][H][W][64] (TO).
template <typename TI, typename TO>
__global__ void k_state_out(const TI* __restrict__ X, const float* __restrict__ scale, TO* __restrict__ dst, Geom g) {
    const size_t per = (size_t)g.H * g.W * NC;
    const size_t n = per * g.B;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        const size_t b = i / per, o = i % per;
        const float v = to_f32<TI>(X[(b * g.state_rows() + g.hx) * g.W * NC + o]) * scale[b * NC + (o & 63)];
        dst[i] = from_f32<TO>(v);
    }
}

// X[b,y,x,c] = img[b,y-py,x-px] * L[c] inside the centred image, 0 in the padding.
template <typename TO>
__global__ void k_lift(const float* __restrict__ img, int ih, int iw, const float* __restrict__ L,
                       TO* __restrict__ X, Geom g) {
    const int py = (g.H - ih) / 2, px = (g.W - iw) / 2;
    const size_t per = (size_t)g.H * g.W * NC;
    const size_t n = per * g.B;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < n; i += (size_t)gridDim.x * blockDim.x) {
        const size_t b = i / per, o = i % per;
        const int c = (int)(o & 63);
        const int x = (int)((o >> 6) % g.W), y = (int)((o >> 6) / g.W);
        const int iy = y - py, ix = x - px;
        float v = 0.f;
        if (iy >= 0 && iy < ih && ix >= 0 && ix < iw) v = img[(b * ih + iy) * iw + ix] * L[c];
        X[(b * g.state_rows() + g.hx) * g.W * NC + o] = from_f32<TO>(v);
    }
}

// field[b][cell] = mean over the 64 channels of the normalised state (stored value x pending scale).  Eight
// threads per cell, eight channels each, summed by a fixed shuffle tree.
template <typename T>
__global__ void __launch_bounds__(256)
k_channel_mean(const T* __restrict__ X, const float* __restrict__ scale, float* __restrict__ field, Geom g) {
    const size_t cells = (size_t)g.H * g.W, n = cells * g.B;
    const int q = threadIdx.x & 7;
    // a warp covers 4 consecutive cells; the loop condition is on the warp's first cell, so all 32 lanes shuffle
    for (size_t i = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) >> 3; (i & ~size_t(3)) < n;
         i += ((size_t)gridDim.x * blockDim.x) >> 3) {
        float s = 0.f;
        const bool live = i < n;
        const size_t b = live ? i / cells : 0, cell = live ? i % cells : 0;
        if (live) {
            const T* px = X + ((b * g.state_rows() + g.hx) * g.W) * NC + cell * NC + q * 8;
#pragma unroll
            for (int k = 0; k < 8; ++k) s = fmaf(to_f32<T>(px[k]), scale[b * NC + q * 8 + k], s);
        }
        s += __shfl_xor_sync(0xffffffffu, s, 1);
        s += __shfl_xor_sync(0xffffffffu, s, 2);
        s += __shfl_xor_sync(0xffffffffu, s, 4);
        if (live && q == 0) field[i] = s * (1.f / NC);
    }
}

// logits[b][o] = sum_c (sums[b][c] * scale[b][c] / cells) Wr[c][o] + br[o]
__global__ void k_pool_readout(const double* __restrict__ sums, const float* __restrict__ scale, double inv_cells,
                               const float* __restrict__ Wr, const float* __restrict__ br, int n_out,
                               float* __restrict__ logits) {
    const int b = blockIdx.x, o = threadIdx.x;
    if (o >= n_out) return;
    double acc = br ? (double)br[o] : 0.0;
    for (int c = 0; c < NC; ++c) acc += sums[b * NC + c] * (double)scale[b * NC + c] * inv_cells * (double)Wr[c * n_out + o];
    logits[b * n_out + o] = (float)acc;
}

}  // namespace slime
