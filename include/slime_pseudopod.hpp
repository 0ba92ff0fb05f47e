// C++ host adapters that put the C ABI of slime_ca.h behind the reference's protocol interfaces.
//
//   SlimePseudopod : ModelProtocol       forward(input, output) = one CA step on device fp32 buffers
//                                        [batch][H][W][64]; effective_rank()/coherence() = results of the last
//                                        compute_fitness().  Chained calls - forward(a, b); forward(b, c); - continue
//                                        the trajectory on the handle without reloading b, so the redistributed value
//                                        of the last two steps stays paired and compute_fitness() works after two
//                                        forwards (set chain_forward = false if b is modified between the calls).
//                                        The only protocol implementer the reference ever had is
//                                        failed_attempts/model.cu:11-59 (Pseudopod : ModelProtocol).
//   SlimeComponent : ComponentProtocol   id / fitness / coherence / hunger bookkeeping around one SlimePseudopod
//                                        (ComponentProtocol and ModelProtocol both name a `coherence` member, so
//                                        one class can not derive from both without ambiguity).
//   SlimeStepKernel : KernelProtocol     launch() enqueues `steps` CA steps of a SlimePseudopod on `stream`.
//
// Header-only; link against libslime_ca.so.
#pragma once
#include <cstdio>
#include <cstring>
#include <stdexcept>
#include <string>

#include "slime_ca.h"
#include "slime_protocols.hpp"

class SlimePseudopod : public ModelProtocol {
public:
    SlimePseudopod(int batch, int height, int width, int n_weight_sets = 1, int dtype = SLIME_CA_F32, int device = 0,
                   float dt = 0.1f) {
        parameters_d = nullptr;   // the handle owns the device copies of the weights
        gradients_d = nullptr;    // the CA is evolved, not trained by gradients
        num_parameters = n_weight_sets * (3 * 8 * 64 * 64 + 512 * 64 + 8 * 9 + 16);
        slime_ca_config cfg{batch, height, width, n_weight_sets, dtype, dt, device, 0, 1};
        const int rc = slime_ca_create(&cfg, &h_);
        if (rc != SLIME_CA_OK) {
            const std::string text = std::string("slime_ca_create: ") + slime_ca_last_error(h_);
            if (h_) slime_ca_destroy(h_);     // create hands the handle back on failure so that the text can be read
            h_ = nullptr;
            throw std::runtime_error(text);
        }
    }
    ~SlimePseudopod() { if (h_) slime_ca_destroy(h_); }
    SlimePseudopod(const SlimePseudopod&) = delete;
    SlimePseudopod& operator=(const SlimePseudopod&) = delete;

    void set_weights(int set, const float* Wp, const float* Wi, const float* Wv, const float* Wo, const float* K,
                     const float* mu, const float* sigma) {
        check(slime_ca_set_weights(h_, set, Wp, Wi, Wv, Wo, K, mu, sigma), "slime_ca_set_weights");
    }

    // ModelProtocol: device fp32 in, device fp32 out, one step
    void forward(float* input, float* output) override {
        if (!(chain_forward && input == last_output_))
            check(slime_ca_set_state_device(h_, input, SLIME_CA_F32, stream), "slime_ca_set_state_device");
        check(slime_ca_step(h_, steps_per_forward, stream), "slime_ca_step");
        check(slime_ca_get_state_device(h_, output, SLIME_CA_F32, stream), "slime_ca_get_state_device");
        last_output_ = output;
    }
    float effective_rank() override { return rank_; }
    float coherence() override { return coherence_; }
    void update_gradients(float) override {}   // no gradient path: weights change by mutation in the caller

    // mean over the batch of rank x coherence of the last two steps
    float compute_fitness() {
        const int b = batch();
        std::string buf(sizeof(float) * 4 * b, '\0');
        float* r = reinterpret_cast<float*>(&buf[0]);
        check(slime_ca_fitness(h_, r, r + b, r + 2 * b, r + 3 * b, stream), "slime_ca_fitness");
        float s[4] = {0, 0, 0, 0};
        for (int k = 0; k < 4; ++k) { for (int i = 0; i < b; ++i) s[k] += r[k * b + i]; s[k] /= b; }
        rank_ = s[0]; coherence_ = s[1]; fitness_ = s[2]; hunger_ = s[3];
        return fitness_;
    }
    float hunger() const { return hunger_; }
    float fitness() const { return fitness_; }
    slime_ca* handle() { return h_; }
    int batch() const { return batch_of(h_); }

    void* stream = nullptr;
    int steps_per_forward = 1;
    bool chain_forward = true;      // forward(in, out) with in == the previous out continues without reloading

private:
    static int batch_of(slime_ca* h) {
        void* p; size_t bytes;
        slime_ca_buffer(h, SLIME_CA_BUF_SCALE, &p, &bytes);
        return (int)(bytes / (64 * sizeof(float)));
    }
    void check(int rc, const char* what) {
        if (rc != SLIME_CA_OK) throw std::runtime_error(std::string(what) + ": " + slime_ca_last_error(h_));
    }
    slime_ca* h_ = nullptr;
    const float* last_output_ = nullptr;
    float rank_ = 0.f, coherence_ = 0.f, fitness_ = 0.f, hunger_ = 1.f;
};

class SlimeComponent : public ComponentProtocol {
public:
    explicit SlimeComponent(SlimePseudopod* model, int component_id = 0) : model_(model) {
        id = component_id;
        reset();
    }
    void reset() override { fitness = 0.f; coherence = 0.f; hunger = 1.f; }
    // "id fitness coherence hunger" as text, the fields failed_attempts/component.cu:28-69 serialised
    void to_dict(char* buffer) override { std::sprintf(buffer, "%d %.9g %.9g %.9g", id, fitness, coherence, hunger); }
    void from_dict(const char* buffer) override { std::sscanf(buffer, "%d %g %g %g", &id, &fitness, &coherence, &hunger); }
    float compute_fitness() override {
        fitness = model_->compute_fitness();
        coherence = model_->coherence();
        hunger = model_->hunger();
        return fitness;
    }

private:
    SlimePseudopod* model_;
};

class SlimeStepKernel : public KernelProtocol {
public:
    SlimeStepKernel(SlimePseudopod* model, int steps) : model_(model), steps_(steps) {
        grid_size = dim3(0, 0, 0);      // the library sizes its own launches (several kernels per step)
        block_size = dim3(256, 1, 1);
        shared_memory = 0;
        stream = nullptr;
    }
    void launch() override {
        if (slime_ca_step(model_->handle(), steps_, stream) != SLIME_CA_OK)
            throw std::runtime_error(slime_ca_last_error(model_->handle()));
    }
    size_t memory_required() const override { return slime_ca_workspace_bytes(model_->handle()); }
    // resident threads per SM of the handle's step kernels over the SM's thread limit, from the occupancy API
    float theoretical_occupancy() const override {
        float o = 0.f;
        if (slime_ca_occupancy(model_->handle(), &o) != SLIME_CA_OK)
            throw std::runtime_error(slime_ca_last_error(model_->handle()));
        return o;
    }

private:
    SlimePseudopod* model_;
    int steps_;
};
