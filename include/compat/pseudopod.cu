// Source-level stand-in for slime/core/pseudopod.cu of J0pari/Slime: put this file in its place (and add this
// repository's include/ to the include path, libslime_ca.so to the link) and slime/core/organism.cu and
// slime/runtime.cu compile unchanged.
//
// What stays: the configuration constants (slime/core/pseudopod.cu:15-21), clamp() (:24-26), the field names and
// order of struct MultiHeadCAState (:29-38), and the names and signatures of the kernels that the step driver
// neural_ca_update_kernel launches from the device (slime/core/organism.cu:642-683) and that
// init_organism_kernel launches (slime/core/organism.cu:926-929).
//
// What changes: the CA step itself no longer runs inside those device-side launches.  A separately linked
// library cannot be entered from a device thread, and the tensor-core step needs host-encoded tensor maps, so
// the three step kernels only RECORD that the driver asked for a generation (SlimeCompatRequest below) and the
// host performs it after the driver kernel has returned: slime_compat_generation() lifts the chemical field
// into the CA (initialize_ca_from_field_kernel, organism.cu:691-720), runs the fused step through the C ABI,
// writes the field back (update_field_from_ca_kernel, organism.cu:723-743) and stores the effective rank where
// compute_effective_rank_kernel was told to (organism.cu:679-683).  run_organism() (slime/runtime.cu:385-414)
// already synchronises once per generation; the call goes right after that synchronisation.
//
// tensor_core_ca_kernel and compute_coherence_kernel (slime/core/pseudopod.cu:256,348) have no caller in the
// live tree and are not provided.
#ifndef PSEUDOPOD_CU
#define PSEUDOPOD_CU

#include <cuda_runtime.h>
#include <cuda_fp16.h>
#include <mma.h>
#include <cooperative_groups.h>
#include <curand_kernel.h>
#include <math.h>
#include <stdint.h>

#include "slime_ca.h"

namespace cg = cooperative_groups;
namespace wmma = nvcuda::wmma;

constexpr int NUM_HEADS = 8;
constexpr int HEAD_DIM = 64;
constexpr int CHANNELS = 512;
constexpr int HIDDEN_DIM = 256;
constexpr int KERNEL_SIZE = 3;
constexpr int GRID_SIZE = 128;
constexpr float MASS_CONSERVATION_EPSILON = 1e-6f;

__device__ __forceinline__ int clamp(int x, int lo, int hi) { return x < lo ? lo : (x > hi ? hi : x); }

struct MultiHeadCAState {
    float* perception_weights;   // [NUM_HEADS][CHANNELS][HIDDEN_DIM]
    float* interaction_weights;  // [NUM_HEADS][CHANNELS][HIDDEN_DIM]
    float* value_weights;        // [NUM_HEADS][HIDDEN_DIM][CHANNELS]
    float* head_mixing_weights;  // [NUM_HEADS][NUM_HEADS]
    float* flow_kernels;         // [NUM_HEADS][3][3]
    float* mass_buffer;
    float* ca_input;
    float* ca_output;
};

// What the device-side launch sites asked for since the host last looked.
struct SlimeCompatRequest {
    int generation_requested;   // multi_head_ca_kernel was launched
    int batch_size, grid_size;  // its arguments
    float dt;                   // flow_lenia_dynamics_kernel's time step
    float* rank_slot;           // compute_effective_rank_kernel's output address (device)
};
__device__ SlimeCompatRequest slime_compat_request;

// The three step kernels: one thread records the request; the launch geometry of the caller does not matter.
__global__ void multi_head_ca_kernel(float* __restrict__, float* __restrict__, float* __restrict__,
                                     float* __restrict__, float* __restrict__, int batch_size, int grid_size) {
    if ((blockIdx.x | blockIdx.y | blockIdx.z | threadIdx.x | threadIdx.y | threadIdx.z) != 0) return;
    slime_compat_request.batch_size = batch_size;
    slime_compat_request.grid_size = grid_size;
    slime_compat_request.generation_requested = 1;
}

__global__ void flow_lenia_dynamics_kernel(float* __restrict__, float* __restrict__, float* __restrict__,
                                           float* __restrict__, int, float dt) {
    if ((blockIdx.x | blockIdx.y | blockIdx.z | threadIdx.x | threadIdx.y | threadIdx.z) != 0) return;
    slime_compat_request.dt = dt;
}

__global__ void mix_heads_kernel(float* __restrict__, float* __restrict__, float* __restrict__, int, int) {}

__global__ void compute_effective_rank_kernel(float* __restrict__, float* __restrict__ effective_rank, int) {
    if ((blockIdx.x | threadIdx.x) != 0) return;
    slime_compat_request.rank_slot = effective_rank;
}

// Weight initialisation, bit-compatible with the reference's (slime/core/pseudopod.cu:386-444) when compiled with the
// reference's flags: thread tid owns subsequence tid of cuRAND's default generator seeded with `seed` and draws, in
// this order, one normal each for element tid of the perception, interaction and value arrays (scaled
// sqrt(2/(fan_in+fan_out)), sqrt(2/CHANNELS), sqrt(2/HIDDEN_DIM)), one normal for mixing element tid < 64
// (identity + 0.01 N) and one uniform for flow tap tid < 72.  The reference then lets threads 0..7 normalise their
// head's nine taps by reading what threads 0..71 wrote, which nothing orders; here the thread of head h replays the
// draws of its nine tap threads itself, so the taps are always the normalised ones.
__device__ __forceinline__ float slime_compat_tap_draw(unsigned int seed, int t) {
    curandState_t rng;
    curand_init(seed, t, 0, &rng);
    curand_normal(&rng); curand_normal(&rng); curand_normal(&rng);      // the three weight draws of thread t
    if (t < NUM_HEADS * NUM_HEADS) curand_normal(&rng);                  // its mixing draw
    return curand_uniform(&rng);
}

__global__ void init_multihead_ca_kernel(MultiHeadCAState* state, unsigned int seed) {
    const int tid = blockIdx.x * blockDim.x + threadIdx.x;
    constexpr int n_big = NUM_HEADS * CHANNELS * HIDDEN_DIM;
    if (tid >= n_big) return;
    curandState_t rng;
    curand_init(seed, tid, 0, &rng);
    state->perception_weights[tid] = curand_normal(&rng) * sqrtf(2.0f / float(CHANNELS + HIDDEN_DIM));
    state->interaction_weights[tid] = curand_normal(&rng) * sqrtf(2.0f / float(CHANNELS));
    state->value_weights[tid] = curand_normal(&rng) * sqrtf(2.0f / float(HIDDEN_DIM));
    if (tid < NUM_HEADS * NUM_HEADS)
        state->head_mixing_weights[tid] = (tid / NUM_HEADS == tid % NUM_HEADS ? 1.0f : 0.0f) + curand_normal(&rng) * 0.01f;
    if (tid < NUM_HEADS) {
        float taps[9], sum = 0.0f;
        for (int t = 0; t < 9; ++t) { taps[t] = slime_compat_tap_draw(seed, tid * 9 + t); sum += taps[t]; }
        for (int t = 0; t < 9; ++t) state->flow_kernels[tid * 9 + t] = taps[t] / sum;
    }
}

// ---- host side ------------------------------------------------------------------------------------------------

// Create the handle for the bundle's grid and upload the bundle's weights (call again after the weights change).
inline int slime_compat_bind(slime_ca** ca, const MultiHeadCAState* dev_state, int dtype, const float* mu,
                             const float* sigma) {
    MultiHeadCAState hs;
    if (cudaMemcpy(&hs, dev_state, sizeof(hs), cudaMemcpyDeviceToHost) != cudaSuccess) return SLIME_CA_ECUDA;
    if (*ca == nullptr) {
        int device = 0;
        cudaGetDevice(&device);
        slime_ca_config cfg{1, GRID_SIZE, GRID_SIZE, 1, dtype, 0.1f, device, 0, 1};
        const int rc = slime_ca_create(&cfg, ca);
        if (rc != SLIME_CA_OK) return rc;
    }
    return slime_ca_set_weights_reference_layout(*ca, 0, hs.perception_weights, hs.interaction_weights,
                                                 hs.value_weights, hs.head_mixing_weights, hs.flow_kernels, mu, sigma);
}

// Perform the generation the device-side launch sites recorded, if any: returns 1 when a generation ran,
// 0 when none was requested, a negative status on error.  `dev_concentration` is the chemical field
// [GRID_SIZE][GRID_SIZE] the driver lifts from and writes back to; `lift` the 64 per-channel lift factors.
inline int slime_compat_generation(slime_ca* ca, float* dev_concentration, const float* lift, int steps,
                                   cudaStream_t stream) {
    SlimeCompatRequest req;
    if (cudaMemcpyFromSymbol(&req, slime_compat_request, sizeof(req)) != cudaSuccess) return -SLIME_CA_ECUDA;
    if (!req.generation_requested) return 0;
    int rc = slime_ca_lift_field_device(ca, dev_concentration, lift, stream);
    if (rc == SLIME_CA_OK) rc = slime_ca_step(ca, steps, stream);
    if (rc == SLIME_CA_OK) rc = slime_ca_field_from_state_device(ca, dev_concentration, stream);
    float rank = 0.f;
    if (rc == SLIME_CA_OK && steps >= 2) {
        rc = slime_ca_fitness(ca, &rank, nullptr, nullptr, nullptr, stream);
        if (rc == SLIME_CA_OK && req.rank_slot &&
            cudaMemcpyAsync(req.rank_slot, &rank, sizeof(float), cudaMemcpyHostToDevice, stream) != cudaSuccess)
            rc = SLIME_CA_ECUDA;
    }
    if (cudaStreamSynchronize(stream) != cudaSuccess) rc = SLIME_CA_ECUDA;
    const SlimeCompatRequest cleared{0, 0, 0, 0.f, nullptr};
    if (cudaMemcpyToSymbol(slime_compat_request, &cleared, sizeof(cleared)) != cudaSuccess) rc = SLIME_CA_ECUDA;
    return rc == SLIME_CA_OK ? 1 : -rc;
}

#endif  // PSEUDOPOD_CU
