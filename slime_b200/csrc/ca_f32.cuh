// fp32 path of the CA step: two SIMT kernels per step, exact expf and division, fp32 FMA accumulation.
// This is the path held to 1e-5 relative L2 against the CPU oracle.
//
//   k1_f32  reads the state with a 1-cell halo, applies the pending per-channel scale, forms for every head
//           the 3x3-convolved input (the stencil commutes with the linear perception projection, so
//           conv_h(X) Wp_h = conv_h(X Wp_h)), projects to U | I | V (64 -> 3x64 per head), applies the growth
//           bell and writes E = exp(G*I) and V, per-head planar [B][8][rows][W][64].
//   k2_f32  reads E with a 2-cell halo and V with a 1-cell halo, Z = box3(E), R = V/Z, V' = E*box3(R)
//           (the closed form of the per-source softmax redistribution), projects concat_h(V') with Wo,
//           writes X+ = scale*X + dt*Y in place and one per-channel partial sum per tile.
// The per-channel renormalisation is lazy: the stored state is un-normalised and the next k1 applies
// scale[b][c] = mass / sum when it loads.
#pragma once
#include "common.cuh"

namespace slime {

constexpr int T32 = 8;                 // tile edge of the fp32 kernels (64 cells)
constexpr int XS32 = 68;               // padded cell stride in floats (keeps float4 alignment, breaks bank ties)
constexpr int K1F32_SMEM = (100 * XS32 + 64 * XS32 + 64 * 192 + 16) * 4;
constexpr int K2F32_SMEM = (144 * 64 + 100 * 64 + 64 * XS32 + 64 * 64 + 2 * 16 * 64) * 4;   // the last term: [16][64] doubles

__global__ void __launch_bounds__(256)
k1_f32(const float* __restrict__ X, const float* __restrict__ scale, const float* __restrict__ Wpiv,
       const float* __restrict__ prm, float* __restrict__ E, float* __restrict__ V, Geom g) {
    extern __shared__ __align__(16) float sm[];
    float* xh = sm;                    // [10*10][XS32]  state halo tile, scale applied
    float* ac = xh + 100 * XS32;       // [64][XS32]     convolved input of the current head
    float* ws = ac + 64 * XS32;        // [64][192]      Wp | Wi | Wv rows of the current head
    float* ps = ws + 64 * 192;         // [PRM]

    const int tid = threadIdx.x;
    const int b = blockIdx.y;
    const int tx0 = (blockIdx.x % g.tiles_x) * T32;
    const int ty0 = (blockIdx.x / g.tiles_x) * T32 - g.he;
    const int set = b / g.per_set;
    const size_t xplane = (size_t)g.state_rows() * g.W * NC;
    const size_t eplane = (size_t)g.ev_rows() * g.W * HD;

    for (int i = tid; i < 100 * 16; i += 256) {
        const int cell = i >> 4, q = i & 15;
        const int r = ty0 + cell / 10 - 1, x = g.wrap_x(tx0 + cell % 10 - 1);
        float4 v = *reinterpret_cast<const float4*>(X + (size_t)b * xplane + ((size_t)g.xrow(r) * g.W + x) * NC + q * 4);
        const float4 s = *reinterpret_cast<const float4*>(scale + b * NC + q * 4);
        v.x *= s.x; v.y *= s.y; v.z *= s.z; v.w *= s.w;
        *reinterpret_cast<float4*>(xh + cell * XS32 + q * 4) = v;
    }

    const int cg = tid >> 4;           // 16 groups of 4 cells (half a tile row each)
    const int d0 = (tid & 15) * 4;     // 4 output dims

    for (int h = 0; h < NH; ++h) {
        __syncthreads();               // previous head done with ac / ws; first pass: xh complete
        const float* wsrc = Wpiv + ((size_t)set * NH + h) * NC * 192;
        for (int i = tid; i < 64 * 192 / 4; i += 256)
            reinterpret_cast<float4*>(ws)[i] = reinterpret_cast<const float4*>(wsrc)[i];
        if (tid < PRM) ps[tid] = prm[((size_t)set * NH + h) * PRM + tid];
        __syncthreads();
        for (int i = tid; i < 64 * 64; i += 256) {
            const int c = i & 63, cell = i >> 6;
            const int cy = cell >> 3, cx = cell & 7;
            float a = 0.f;
#pragma unroll
            for (int t = 0; t < 9; ++t)
                a = fmaf(ps[t], xh[((cy + t / 3) * 10 + cx + t % 3) * XS32 + c], a);
            ac[cell * XS32 + c] = a;
        }
        __syncthreads();

        float u[4][4], iv[4][4], vv[4][4];
#pragma unroll
        for (int j = 0; j < 4; ++j)
#pragma unroll
            for (int k = 0; k < 4; ++k) u[j][k] = iv[j][k] = vv[j][k] = 0.f;

        for (int k4 = 0; k4 < 16; ++k4) {
            float4 a4[4], x4[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) {
                const int cell = cg * 4 + j;
                a4[j] = *reinterpret_cast<const float4*>(ac + cell * XS32 + k4 * 4);
                x4[j] = *reinterpret_cast<const float4*>(xh + (((cell >> 3) + 1) * 10 + (cell & 7) + 1) * XS32 + k4 * 4);
            }
#pragma unroll
            for (int kk = 0; kk < 4; ++kk) {
                const float* wr = ws + (k4 * 4 + kk) * 192 + d0;
                const float4 wp = *reinterpret_cast<const float4*>(wr);
                const float4 wi = *reinterpret_cast<const float4*>(wr + 64);
                const float4 wv = *reinterpret_cast<const float4*>(wr + 128);
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float a = kk == 0 ? a4[j].x : kk == 1 ? a4[j].y : kk == 2 ? a4[j].z : a4[j].w;
                    const float x = kk == 0 ? x4[j].x : kk == 1 ? x4[j].y : kk == 2 ? x4[j].z : x4[j].w;
                    u[j][0] = fmaf(a, wp.x, u[j][0]); u[j][1] = fmaf(a, wp.y, u[j][1]);
                    u[j][2] = fmaf(a, wp.z, u[j][2]); u[j][3] = fmaf(a, wp.w, u[j][3]);
                    iv[j][0] = fmaf(x, wi.x, iv[j][0]); iv[j][1] = fmaf(x, wi.y, iv[j][1]);
                    iv[j][2] = fmaf(x, wi.z, iv[j][2]); iv[j][3] = fmaf(x, wi.w, iv[j][3]);
                    vv[j][0] = fmaf(x, wv.x, vv[j][0]); vv[j][1] = fmaf(x, wv.y, vv[j][1]);
                    vv[j][2] = fmaf(x, wv.z, vv[j][2]); vv[j][3] = fmaf(x, wv.w, vv[j][3]);
                }
            }
        }

        const float mu = ps[9], nis = ps[10];
#pragma unroll
        for (int j = 0; j < 4; ++j) {
            const int cell = cg * 4 + j;
            const int r = ty0 + (cell >> 3), x = tx0 + (cell & 7);
            if (r >= g.H + g.he || x >= g.W) continue;
            float4 e, vo;
            float* ep = &e.x;
            float* vp = &vo.x;
#pragma unroll
            for (int k = 0; k < 4; ++k) {
                const float z = u[j][k] - mu;
                const float gr = 2.f * expf(z * z * nis) - 1.f;
                ep[k] = expf(fminf(fmaxf(gr * iv[j][k], -ACT_CLAMP), ACT_CLAMP));
                vp[k] = vv[j][k];
            }
            const size_t o = ((size_t)b * NH + h) * eplane + ((size_t)g.erow(r) * g.W + x) * HD + d0;
            *reinterpret_cast<float4*>(E + o) = e;
            *reinterpret_cast<float4*>(V + o) = vo;
        }
    }
}

__global__ void __launch_bounds__(256)
k2_f32(float* __restrict__ X, const float* __restrict__ scale, const float* __restrict__ Wo,
       const float* __restrict__ E, const float* __restrict__ V, float* __restrict__ partial, size_t lo_offset,
       float* __restrict__ vprime, Geom g) {
    extern __shared__ __align__(16) float sm[];
    float* es = sm;                    // [12*12][64]  E with a 2-cell halo
    float* vs = es + 144 * 64;         // [10*10][64]  V, then R = V / box3(E), with a 1-cell halo
    float* vp = vs + 100 * 64;         // [64][XS32]   V' of the tile
    float* wo = vp + 64 * XS32;        // [64][64]     Wo rows of the current head
    double* red = reinterpret_cast<double*>(wo + 64 * 64);   // [16][64] fp64 (the offset is a multiple of 8 bytes)

    const int tid = threadIdx.x;
    const int b = blockIdx.y;
    const int tx0 = (blockIdx.x % g.tiles_x) * T32;
    const int ty0 = (blockIdx.x / g.tiles_x) * T32;
    const int set = b / g.per_set;
    const size_t xplane = (size_t)g.state_rows() * g.W * NC;
    const size_t eplane = (size_t)g.ev_rows() * g.W * HD;
    const size_t vplane = (size_t)g.H * g.W * HD;
    const int cg = tid >> 4;
    const int c0 = (tid & 15) * 4;

    float acc[4][4];
#pragma unroll
    for (int j = 0; j < 4; ++j)
#pragma unroll
        for (int k = 0; k < 4; ++k) acc[j][k] = 0.f;

    for (int h = 0; h < NH; ++h) {
        const float* Eh = E + ((size_t)b * NH + h) * eplane;
        const float* Vh = V + ((size_t)b * NH + h) * eplane;
        __syncthreads();
        for (int i = tid; i < 144 * 16; i += 256) {
            const int cell = i >> 4, q = i & 15;
            const int r = ty0 + cell / 12 - 2, x = g.wrap_x(tx0 + cell % 12 - 2);
            reinterpret_cast<float4*>(es)[i] =
                *reinterpret_cast<const float4*>(Eh + ((size_t)g.erow(r) * g.W + x) * HD + q * 4);
        }
        for (int i = tid; i < 100 * 16; i += 256) {
            const int cell = i >> 4, q = i & 15;
            const int r = ty0 + cell / 10 - 1, x = g.wrap_x(tx0 + cell % 10 - 1);
            reinterpret_cast<float4*>(vs)[i] =
                *reinterpret_cast<const float4*>(Vh + ((size_t)g.erow(r) * g.W + x) * HD + q * 4);
        }
        const float* wsrc = Wo + ((size_t)set * NH + h) * HD * NC;
        for (int i = tid; i < 64 * 64 / 4; i += 256)
            reinterpret_cast<float4*>(wo)[i] = reinterpret_cast<const float4*>(wsrc)[i];
        __syncthreads();
        // R = V / box3(E) on the 10x10 ring-extended tile (each item owns its own 4 values: in place)
        for (int i = tid; i < 100 * 16; i += 256) {
            const int cell = i >> 4, q = i & 15;
            const int vy = cell / 10, vx = cell % 10;
            float4 z = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
            for (int t = 0; t < 9; ++t) {
                const float4 e = *reinterpret_cast<const float4*>(es + ((vy + t / 3) * 12 + vx + t % 3) * 64 + q * 4);
                z.x += e.x; z.y += e.y; z.z += e.z; z.w += e.w;
            }
            float4 v = reinterpret_cast<float4*>(vs)[i];
            v.x /= z.x; v.y /= z.y; v.z /= z.z; v.w /= z.w;
            reinterpret_cast<float4*>(vs)[i] = v;
        }
        __syncthreads();
        // V' = E * box3(R) on the 8x8 tile
        for (int i = tid; i < 64 * 16; i += 256) {
            const int cell = i >> 4, q = i & 15;
            const int cy = cell >> 3, cx = cell & 7;
            float4 s = make_float4(0.f, 0.f, 0.f, 0.f);
#pragma unroll
            for (int t = 0; t < 9; ++t) {
                const float4 r = *reinterpret_cast<const float4*>(vs + ((cy + t / 3) * 10 + cx + t % 3) * 64 + q * 4);
                s.x += r.x; s.y += r.y; s.z += r.z; s.w += r.w;
            }
            const float4 e = *reinterpret_cast<const float4*>(es + ((cy + 2) * 12 + cx + 2) * 64 + q * 4);
            s.x *= e.x; s.y *= e.y; s.z *= e.z; s.w *= e.w;
            *reinterpret_cast<float4*>(vp + cell * XS32 + q * 4) = s;
            if (vprime != nullptr && ty0 + cy < g.H && tx0 + cx < g.W)
                *reinterpret_cast<float4*>(vprime + ((size_t)b * NH + h) * vplane +
                                           ((size_t)(ty0 + cy) * g.W + tx0 + cx) * HD + q * 4) = s;
        }
        __syncthreads();
        for (int k4 = 0; k4 < 16; ++k4) {
            float4 a4[4];
#pragma unroll
            for (int j = 0; j < 4; ++j) a4[j] = *reinterpret_cast<const float4*>(vp + (cg * 4 + j) * XS32 + k4 * 4);
#pragma unroll
            for (int kk = 0; kk < 4; ++kk) {
                const float4 w = *reinterpret_cast<const float4*>(wo + (k4 * 4 + kk) * 64 + c0);
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    const float a = kk == 0 ? a4[j].x : kk == 1 ? a4[j].y : kk == 2 ? a4[j].z : a4[j].w;
                    acc[j][0] = fmaf(a, w.x, acc[j][0]); acc[j][1] = fmaf(a, w.y, acc[j][1]);
                    acc[j][2] = fmaf(a, w.z, acc[j][2]); acc[j][3] = fmaf(a, w.w, acc[j][3]);
                }
            }
        }
    }

    // X+ = scale * X + dt * Y, in place, and the tile's per-channel sums of what was stored
    const float4 s = *reinterpret_cast<const float4*>(scale + b * NC + c0);
    // The tile's channel sums are kept in fp64 and handed on as a float pair (value, remainder): a state that has
    // grown large and signed makes the per-channel sum a small difference of large terms, and fp32 tile sums would
    // then miss the 1e-6 bound on the renormalised mass.
    double psum[4] = {0.0, 0.0, 0.0, 0.0};
#pragma unroll
    for (int j = 0; j < 4; ++j) {
        const int cell = cg * 4 + j;
        const int r = ty0 + (cell >> 3), x = tx0 + (cell & 7);
        if (r >= g.H || x >= g.W) continue;
        float* px = X + (size_t)b * xplane + ((size_t)g.xrow(r) * g.W + x) * NC + c0;
        float4 v = *reinterpret_cast<const float4*>(px);
        v.x = fmaf(g.dt, acc[j][0], v.x * s.x); v.y = fmaf(g.dt, acc[j][1], v.y * s.y);
        v.z = fmaf(g.dt, acc[j][2], v.z * s.z); v.w = fmaf(g.dt, acc[j][3], v.w * s.w);
        *reinterpret_cast<float4*>(px) = v;
        psum[0] += (double)v.x; psum[1] += (double)v.y; psum[2] += (double)v.z; psum[3] += (double)v.w;
    }
#pragma unroll
    for (int k = 0; k < 4; ++k) red[cg * 64 + c0 + k] = psum[k];
    __syncthreads();
    if (tid < 64) {
        double t = 0.0;
#pragma unroll
        for (int k = 0; k < 16; ++k) t += red[k * 64 + tid];
        const size_t o = ((size_t)b * gridDim.x + blockIdx.x) * NC + tid;
        const float hi = (float)t;
        partial[o] = hi;
        partial[o + lo_offset] = (float)(t - (double)hi);
    }
}

}  // namespace slime
