// Shared definitions of the CA step kernels (sm_100a only).
#pragma once
#include <cuda_bf16.h>
#include <cuda_runtime.h>
#include <stdint.h>

namespace slime {

constexpr int NH = 8;    // heads            (slime/core/pseudopod.cu:15)
constexpr int HD = 64;   // head dim         (slime/core/pseudopod.cu:16)
constexpr int NC = 64;   // state channels
constexpr int HC = NH * HD;
// The activation A = G * I is clamped to +-ACT_CLAMP before E = exp(A): the redistribution is evaluated in its
// closed form, without the softmax's max-subtraction, and exp(80) = 5.5e34 keeps nine-term sums finite in fp32.
// The clamp is part of the step's definition (the CPU oracle applies the same one).
constexpr float ACT_CLAMP = 80.f;
constexpr int PRM = 12;  // floats per head in the parameter block: 9 taps, mu, -1/(2 sigma^2), pad

// Geometry of one launch.  Rows are addressed in "own" coordinates r: 0..H-1 are the rows this handle owns.
// Torus mode wraps r modulo H.  Stripe mode has hx halo rows above and below the own rows in the state
// buffer and he halo rows in the E/V intermediates, and never wraps in y; x always wraps.
struct Geom {
    int B, H, W;
    int hx, he;      // halo rows of the state / of the intermediates (0,0 torus; 3,2 stripe)
    int wrap_y;      // 1 = torus in y
    int per_set;     // grids per weight set
    int tiles_x;     // tiles per row of tiles
    int ev_h, ev_w;  // rows and columns of one E/V plane.  fp32 path: H + 2*he rows of W cells.  bf16 path: the
                     // plane carries a 2-cell apron all around, (H + 4) x (W + 4), holding wrapped copies (or, in
                     // stripe mode, the computed halo rows), so the second kernel reads it without any wrap logic
    float dt;

    __host__ __device__ int state_rows() const { return H + 2 * hx; }
    __host__ __device__ int ev_rows() const { return ev_h; }
    __device__ int wrap_x(int x) const { x %= W; return x < 0 ? x + W : x; }
    // physical row in the state buffer of own-coordinate row r
    __device__ int xrow(int r) const {
        if (wrap_y) { r %= H; return r < 0 ? r + H : r; }
        r = r < -hx ? -hx : (r > H + hx - 1 ? H + hx - 1 : r);
        return r + hx;
    }
    // physical row in an E/V plane of own-coordinate row r
    __device__ int erow(int r) const {
        if (wrap_y) { r %= H; return r < 0 ? r + H : r; }
        r = r < -he ? -he : (r > H + he - 1 ? H + he - 1 : r);
        return r + he;
    }
};

__device__ __forceinline__ float bf16_lo(uint32_t v) { return __uint_as_float(v << 16); }
__device__ __forceinline__ float bf16_hi(uint32_t v) { return __uint_as_float(v & 0xffff0000u); }
__device__ __forceinline__ uint32_t pack_bf16(float lo, float hi) {
    __nv_bfloat162 p = __floats2bfloat162_rn(lo, hi);
    return *reinterpret_cast<uint32_t*>(&p);
}

}  // namespace slime
