// The population step that consumes the fitness scalars: culling, selection of the best weight set, and refilling
// every culled slot with a mutated copy of it, all on the device-resident fp32 master copy of the weights; plus
// the kernel that turns master weights into the operand layouts the step kernels read.
//
// Rules, as the reference states them for its component pool:
//   culled  : fitness < 0.1 * fitness_threshold, or hunger > hunger_threshold   (slime/core/organism.cu:594-611)
//   best    : highest fitness among the survivors                                (slime/core/organism.cu:442-470)
//   refill  : copy of the parent, each value perturbed with probability mutation_rate by a normal draw
//             (slime/memory/pool.cu:84-93; the driver passes rate 0.01, slime/core/organism.cu:574-579)
// A weight set's fitness / hunger is the mean over its grids.  The perturbations come from a counter hash of
// (seed, generation, set, value index): any launch geometry gives the same population.
#pragma once
#include "common.cuh"

namespace slime {

// master copy of one weight set (fp32): Wp | Wi | Wv [8][64][64], Wo [512][64], K [8][9], mu [8], sigma [8]
constexpr int MW_WP = 0, MW_WI = 32768, MW_WV = 65536, MW_WO = 98304, MW_K = 131072, MW_MU = 131144, MW_SIGMA = 131152;
constexpr int MW_MUTABLE = 131072;   // the four matrices mutate; taps, mu and sigma are inherited unchanged
constexpr int MW_STRIDE = 131168;    // floats per set, a multiple of 32

struct EvolveParams {
    float fitness_threshold, hunger_threshold, mutation_rate, mutation_sigma;
    unsigned long long seed;
    int generation;
};

__host__ __device__ __forceinline__ uint64_t evolve_mix(uint64_t z) {
    z += 0x9e3779b97f4a7c15ull;
    z = (z ^ (z >> 30)) * 0xbf58476d1ce4e5b9ull;
    z = (z ^ (z >> 27)) * 0x94d049bb133111ebull;
    return z ^ (z >> 31);
}
// draw k (0, 1, 2) of value i of set s: 24 random bits
__host__ __device__ __forceinline__ uint32_t evolve_bits(uint64_t seed, int generation, int s, int i, int k) {
    const uint64_t key = evolve_mix(evolve_mix(seed ^ ((uint64_t)(uint32_t)generation << 32)) ^ (uint64_t)(uint32_t)s);
    return (uint32_t)(evolve_mix(key ^ ((uint64_t)(uint32_t)i * 4u + (uint32_t)k)) >> 40);
}

// One block.  set_stats[s] = {mean fitness, mean hunger}; parent[s] = s for survivors, the best survivor for
// culled sets (or s itself when nothing survives); info = {best or -1, number of replaced sets}.
__global__ void __launch_bounds__(256)
k_evolve_select(const float* __restrict__ fit, int n_sets, int per_set, EvolveParams p, float* __restrict__ set_stats,
                int* __restrict__ parent, int* __restrict__ info) {
    __shared__ int s_best;
    for (int s = threadIdx.x; s < n_sets; s += blockDim.x) {
        double f = 0.0, q = 0.0;
        for (int j = 0; j < per_set; ++j) {
            f += (double)fit[(size_t)(s * per_set + j) * 4 + 2];
            q += (double)fit[(size_t)(s * per_set + j) * 4 + 3];
        }
        const float mf = (float)(f / per_set), mq = (float)(q / per_set);
        set_stats[2 * s] = mf;
        set_stats[2 * s + 1] = mq;
        const bool alive = isfinite(mf) && isfinite(mq) && !(mf < 0.1f * p.fitness_threshold) && !(mq > p.hunger_threshold);
        parent[s] = alive ? s : -1;
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int best = -1, replaced = 0;
        for (int s = 0; s < n_sets; ++s) {
            if (parent[s] < 0) { ++replaced; continue; }
            if (best < 0 || set_stats[2 * s] > set_stats[2 * best]) best = s;
        }
        s_best = best;
        info[0] = best;
        info[1] = best < 0 ? 0 : replaced;
    }
    __syncthreads();
    const int best = s_best;
    for (int s = threadIdx.x; s < n_sets; s += blockDim.x)
        if (parent[s] < 0) parent[s] = best < 0 ? s : best;
}

// grid (blocks, n_sets): culled sets become perturbed copies of their parent (which is a survivor and is not
// written in this launch).
__global__ void __launch_bounds__(256)
k_evolve_refill(float* __restrict__ master, const int* __restrict__ parent, EvolveParams p) {
    const int s = blockIdx.y, par = parent[s];
    if (par == s) return;
    const float* src = master + (size_t)par * MW_STRIDE;
    float* dst = master + (size_t)s * MW_STRIDE;
    const uint32_t rate24 = (uint32_t)(fminf(fmaxf(p.mutation_rate, 0.f), 1.f) * 16777216.0f);
    for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < MW_STRIDE; i += gridDim.x * blockDim.x) {
        float v = src[i];
        if (i < MW_MUTABLE && evolve_bits(p.seed, p.generation, s, i, 0) < rate24) {
            const float u1 = ((float)evolve_bits(p.seed, p.generation, s, i, 1) + 1.0f) * (1.0f / 16777216.0f);   // (0, 1]
            const float u2 = (float)evolve_bits(p.seed, p.generation, s, i, 2) * (1.0f / 16777216.0f);
            v += p.mutation_sigma * sqrtf(-2.0f * logf(u1)) * cosf(6.283185307179586f * u2);
        }
        dst[i] = v;
    }
}

// grid (blocks, n_sets): master weights -> the layouts the step kernels read.  `only`, when given, restricts the
// work to sets whose parent differs from themselves (the ones the refill just rewrote).
//   fp32 path: wpiv [set][8][64 c][192] = Wp | Wi | Wv rows, wo [set][512][64] as stored, prm {taps, mu, -1/(2 sigma^2)}
//   bf16 path: w1 [set][8][192 rows = output column][64 c] with Wp scaled by s = sqrt(log2(e) / (2 sigma^2)) and
//              Wi by log2(e), wo [set][8][64 c][64 d], prm {taps, mu * s, s}
__global__ void __launch_bounds__(256)
k_weights_layout(const float* __restrict__ master, const int* __restrict__ only, int first_set, int bf16,
                 float* __restrict__ wpiv_f32, float* __restrict__ wo_f32, __nv_bfloat16* __restrict__ w1_bf16,
                 __nv_bfloat16* __restrict__ wo_bf16, float* __restrict__ prm) {
    const int s = first_set + blockIdx.y;
    if (only != nullptr && only[s] == s) return;
    const float* m = master + (size_t)s * MW_STRIDE;
    const int t0 = blockIdx.x * blockDim.x + threadIdx.x, nt = gridDim.x * blockDim.x;
    if (t0 < NH) {
        const int hd = t0;
        const float mu = m[MW_MU + hd], sg = m[MW_SIGMA + hd];
        float* q = prm + ((size_t)s * NH + hd) * PRM;
        for (int t = 0; t < 9; ++t) q[t] = m[MW_K + hd * 9 + t];
        if (bf16) {
            const float sc = sqrtf(1.4426950408889634f / (2.f * sg * sg));
            q[9] = mu * sc; q[10] = sc;
        } else {
            q[9] = mu; q[10] = -1.f / (2.f * sg * sg);
        }
        q[11] = 0.f;
    }
    for (int i = t0; i < NH * NC * HD; i += nt) {
        const int hd = i >> 12, c = (i >> 6) & 63, d = i & 63;   // source index [hd][c][d]; for Wo: [hd][d'=c][c'=d]
        if (bf16) {
            const float sg = m[MW_SIGMA + hd];
            const float sc = sqrtf(1.4426950408889634f / (2.f * sg * sg));
            __nv_bfloat16* w1 = w1_bf16 + (size_t)s * NH * 192 * 64;
            w1[((size_t)hd * 192 + d) * 64 + c] = __float2bfloat16_rn(m[MW_WP + i] * sc);
            w1[((size_t)hd * 192 + 64 + d) * 64 + c] = __float2bfloat16_rn(m[MW_WI + i] * 1.4426950408889634f);
            w1[((size_t)hd * 192 + 128 + d) * 64 + c] = __float2bfloat16_rn(m[MW_WV + i]);
            // Wo[(hd*64 + d')][c'] -> row c' (output channel), column d'
            wo_bf16[(size_t)s * NH * 64 * 64 + ((size_t)hd * 64 + d) * 64 + c] = __float2bfloat16_rn(m[MW_WO + i]);
        } else {
            float* w = wpiv_f32 + (size_t)s * NH * NC * 192 + ((size_t)hd * NC + c) * 192 + d;
            w[0] = m[MW_WP + i]; w[64] = m[MW_WI + i]; w[128] = m[MW_WV + i];
            wo_f32[(size_t)s * NH * HD * NC + i] = m[MW_WO + i];
        }
    }
}

}  // namespace slime
