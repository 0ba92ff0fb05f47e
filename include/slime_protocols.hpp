// Abstract protocol structs of J0pari/Slime, declared with the member order and virtual-function order of the
// originals so that objects are interchangeable with code compiled against them:
//   KernelProtocol     slime/proto/kernel.cu:6-15
//   ModelProtocol      slime/proto/model.cu:5-14
//   ComponentProtocol  slime/proto/component.cu:5-15
//   MemoryProtocol     slime/proto/memory.cu:5-15
// A translation unit that already includes the reference's own proto/*.cu defines SLIME_HAVE_REFERENCE_PROTOCOLS
// and this header then declares nothing.
#pragma once
#include <cuda_runtime.h>

#include <cstddef>

#ifndef SLIME_HAVE_REFERENCE_PROTOCOLS

struct KernelProtocol {
    dim3 grid_size;
    dim3 block_size;
    size_t shared_memory;
    cudaStream_t stream;

    virtual void launch() = 0;
    virtual size_t memory_required() const = 0;
    virtual float theoretical_occupancy() const = 0;
};

struct ModelProtocol {
    float* parameters_d;
    float* gradients_d;
    int num_parameters;

    virtual void forward(float* input, float* output) = 0;
    virtual float effective_rank() = 0;
    virtual float coherence() = 0;
    virtual void update_gradients(float learning_rate) = 0;
};

struct ComponentProtocol {
    int id;
    float fitness;
    float coherence;
    float hunger;

    virtual void reset() = 0;
    virtual void to_dict(char* buffer) = 0;
    virtual void from_dict(const char* buffer) = 0;
    virtual float compute_fitness() = 0;
};

struct MemoryProtocol {
    float* memories_d;
    float* decay_factors_d;
    int capacity;
    float decay_rate;

    virtual void store(float* data, int size) = 0;
    virtual void recall(float* output, float* weights) = 0;
    virtual void apply_decay(float timestep) = 0;
    virtual size_t memory_bytes() const = 0;
};

#endif  // SLIME_HAVE_REFERENCE_PROTOCOLS
