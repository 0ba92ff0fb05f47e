// C ABI of the B200 Flow-Lenia CA step (see include/slime_ca.h): handle, buffers, launch sequencing.
// Host-side step driver: what neural_ca_update_kernel (slime/core/organism.cu:617-688) does from a device
// thread with dynamic parallelism is sequenced here from the host on one stream.
#include "../../include/slime_ca.h"

#include <atomic>
#include <cstdio>
#include <cstdlib>
#include <cstring>
#include <new>
#include <string>
#include <vector>

#include "ca_aux.cuh"
#include "ca_bf16.cuh"
#include "ca_f32.cuh"
#include "common.cuh"
#include "fitness.cuh"
#include "evolve.cuh"
#include "ring.cuh"

#include <chrono>
#include <thread>

using namespace slime;

struct slime_ca {
    slime_ca_config cfg{};
    Geom g{};
    size_t esz = 4;                 // bytes per stored element
    void* X = nullptr;              // [B][H+2hx][W][64]
    void* E = nullptr;              // [B][8][ev_h][ev_w][64] (see Geom)
    void* V = nullptr;
    void* vprime[2] = {nullptr, nullptr};
    int vp_last = 0;                // index of the buffer holding the most recent V'
    long long steps_done = 0, vp_steps = 0;
    float* scale = nullptr;
    double* mass = nullptr;
    double* sums = nullptr;
    float* partial = nullptr;
    int partial_cap = 0;
    size_t partial_lo = 0;          // fp32 path: offset (floats) of the remainders of the step's tile sums
    double* seg_sums = nullptr;
    int* tickets = nullptr;          // one per grid: blocks of the reduction that have finished (back at 0 after each launch)
    int k1_tiles = 0, k2_tiles = 0, tiles_x = 0;
    // weights
    float* wpiv_f32 = nullptr;      // [sets][8][64][192]  rows c_in, columns Wp | Wi | Wv
    float* wo_f32 = nullptr;        // [sets][8][64][64]   rows d, columns c_out
    float* prm = nullptr;           // [sets][8][PRM]
    __nv_bfloat16* w1_bf16 = nullptr;  // [sets][8][192][64]  rows = output column (Wp|Wi|Wv), K = c_in contiguous
    __nv_bfloat16* wo_bf16 = nullptr;  // [sets][8][64][64]   rows = c_out, K = d contiguous
    float* master = nullptr;        // [sets][MW_STRIDE] fp32 master copy in the upload's own index order
    float* set_stats = nullptr;     // [sets][2] mean fitness, mean hunger of the last population step
    int* parent = nullptr;          // [sets] parent of each set after the last population step
    int* evolve_info = nullptr;     // {best set, replaced sets}
    std::vector<char> weights_set;
    bool state_set = false;
    bool fitness_valid = false;     // fit_dev holds the fitness of the current V' pair
    bool evolved = false;           // `parent` holds the result of a population step
    // fitness scratch
    double* gram_part = nullptr;
    int gram_splits = 0;
    CUtensorMap gram_map[2];        // bf16 path: tensor maps over the two V' buffers for the tensor-core Gram
    float* head_rank = nullptr;
    double* pearson_part = nullptr;
    int pearson_splits = 0;
    float* fit_dev = nullptr;
    int* dev_status = nullptr;      // status word kernels with bounded waits report into
    int* host_status = nullptr;     // pinned host mirror of it: copied back behind every batch of steps, read without
                                    // synchronising at the start of the next call
    // row-stripe ring (stripe mode): NCCL communicator over the ranks that hold the other stripes
    void* comm = nullptr;
    bool own_comm = false;
    int ring_rank = 0, ring_world = 0;   // world 0 = no ring attached
    size_t bytes = 0;
    long long launches = 0;
    std::string err = "";
    Bf16Plan bf{};
};

namespace {

int fail(slime_ca* h, int code, const std::string& msg) {
    if (h) h->err = msg;
    return code;
}

#define CK(h, call)                                                                                   \
    do {                                                                                              \
        cudaError_t e_ = (call);                                                                      \
        if (e_ != cudaSuccess)                                                                        \
            return fail(h, SLIME_CA_ECUDA, std::string(#call) + ": " + cudaGetErrorString(e_));       \
    } while (0)

#define LAUNCHED(h)                                                                                   \
    do {                                                                                              \
        ++(h)->launches;                                                                              \
        cudaError_t e_ = cudaGetLastError();                                                          \
        if (e_ != cudaSuccess)                                                                        \
            return fail(h, SLIME_CA_ECUDA, std::string("kernel launch: ") + cudaGetErrorString(e_));  \
    } while (0)

template <typename T>
int dev_alloc(slime_ca* h, T** p, size_t n) {
    void* q = nullptr;
    cudaError_t e = cudaMalloc(&q, n * sizeof(T));
    if (e != cudaSuccess) {
        cudaGetLastError();
        return fail(h, SLIME_CA_ENOMEM, "cudaMalloc of " + std::to_string(n * sizeof(T)) + " bytes: " + cudaGetErrorString(e));
    }
    h->bytes += n * sizeof(T);
    *p = static_cast<T*>(q);
    return SLIME_CA_OK;
}

int grid_for(size_t n) {
    size_t b = (n + 255) / 256;
    return (int)(b > 148 * 16 ? 148 * 16 : (b ? b : 1));
}

bool is_bf16(const slime_ca* h) { return h->cfg.dtype == SLIME_CA_BF16; }

// sums <- per-channel sums of the stored state's own rows; mode as in k_finish_sums
int channel_sums(slime_ca* h, int mode, cudaStream_t st) {
    const size_t cells = (size_t)h->g.H * h->g.W;
    const int chunks = (int)((cells + 255) / 256);
    dim3 grid(chunks, h->g.B);
    // a fresh state also starts the reduction's tickets afresh (they are only non-zero if a launch before was cut short)
    CK(h, cudaMemsetAsync(h->tickets, 0, (size_t)h->g.B * sizeof(int), st));
    if (is_bf16(h)) k_channel_partials<__nv_bfloat16><<<grid, 256, 0, st>>>((const __nv_bfloat16*)h->X, h->partial, h->g);
    else k_channel_partials<float><<<grid, 256, 0, st>>>((const float*)h->X, h->partial, h->g);
    LAUNCHED(h);
    const int nseg = chunks < 64 ? chunks : 64;
    k_reduce_finish<<<dim3(nseg, h->g.B), 256, 0, st>>>(h->partial, chunks, h->seg_sums, 0, h->tickets, h->sums, h->mass,
                                                        h->scale, mode);
    LAUNCHED(h);
    return SLIME_CA_OK;
}

// the kernels of one step up to and including BUF_SUMS; `emit` = V' destination or null
// `ev`, when given, receives three records: before k1, between k1 and k2, after k2.  sums_mode 2 also sets the new
// scale from the local sums (a caller that all-reduces the sums first passes 0 and sets the scale afterwards)
int step_kernels(slime_ca* h, void* emit, cudaStream_t st, cudaEvent_t* ev = nullptr, int sums_mode = 0) {
    const Geom& g = h->g;
    if (ev) CK(h, cudaEventRecord(ev[0], st));
    if (is_bf16(h)) {
        if (bf16_k1(h->bf, (const __nv_bfloat16*)h->X, h->scale, h->prm, (__nv_bfloat16*)h->E, (__nv_bfloat16*)h->V,
                    h->dev_status, g, st) != 0)
            return fail(h, SLIME_CA_ECUDA, std::string("bf16 k1 launch: ") + cudaGetErrorString(cudaGetLastError()));
        ++h->launches;
        if (ev) CK(h, cudaEventRecord(ev[1], st));
        if (bf16_k2(h->bf, (__nv_bfloat16*)h->X, h->scale, (const __nv_bfloat16*)h->E, (const __nv_bfloat16*)h->V,
                    h->partial, (__nv_bfloat16*)emit, h->dev_status, g, st) != 0)
            return fail(h, SLIME_CA_ECUDA, std::string("bf16 k2 launch: ") + cudaGetErrorString(cudaGetLastError()));
        ++h->launches;
    } else {
        k1_f32<<<dim3(h->k1_tiles, g.B), 256, K1F32_SMEM, st>>>((const float*)h->X, h->scale, h->wpiv_f32, h->prm,
                                                                 (float*)h->E, (float*)h->V, g);
        LAUNCHED(h);
        if (ev) CK(h, cudaEventRecord(ev[1], st));
        k2_f32<<<dim3(h->k2_tiles, g.B), 256, K2F32_SMEM, st>>>((float*)h->X, h->scale, h->wo_f32, (const float*)h->E,
                                                                 (const float*)h->V, h->partial, h->partial_lo, (float*)emit, g);
        LAUNCHED(h);
    }
    if (ev) CK(h, cudaEventRecord(ev[2], st));
    const int nseg = h->k2_tiles < 64 ? h->k2_tiles : 64;
    k_reduce_finish<<<dim3(nseg, g.B), 256, 0, st>>>(h->partial, h->k2_tiles, h->seg_sums, is_bf16(h) ? 0 : h->partial_lo,
                                                     h->tickets, h->sums, h->mass, h->scale, sums_mode);
    LAUNCHED(h);
    return SLIME_CA_OK;
}

int ready(slime_ca* h) {
    if (!h) return SLIME_CA_EINVAL;
    for (char c : h->weights_set)
        if (!c) return fail(h, SLIME_CA_ESTATE, "not every weight set has been uploaded");
    if (!h->state_set) return fail(h, SLIME_CA_ESTATE, "no state has been loaded");
    return SLIME_CA_OK;
}

void ring_release(slime_ca* h) {
    if (h->comm && h->own_comm && nccl::api().ok) nccl::api().CommDestroy((nccl::comm_t)h->comm);
    h->comm = nullptr;
    h->own_comm = false;
    h->ring_world = 0;
}

#define NK(h, call)                                                                                         \
    do {                                                                                                    \
        int r_ = (call);                                                                                    \
        if (r_ != nccl::SUCCESS)                                                                            \
            return fail(h, SLIME_CA_ECOMM, std::string(#call) + ": " + nccl::describe(r_));                 \
    } while (0)

// Refresh the 3 + 3 halo rows of every grid's stripe from the ring neighbours' own rows (the step's dependency
// radius is 3 rows).  Rows travel straight between the state buffers: my top own rows land in the upper
// neighbour's bottom halo, my bottom own rows in the lower neighbour's top halo; with one rank the stripe wraps
// onto itself by device copies.  Everything is enqueued on `st`; nothing synchronises.
int ring_exchange(slime_ca* h, cudaStream_t st) {
    const Geom& g = h->g;
    const size_t row = (size_t)g.W * NC * h->esz, halo = 3 * row, plane = (size_t)g.state_rows() * row;
    char* X = static_cast<char*>(h->X);
    if (h->ring_world == 1) {
        for (int b = 0; b < g.B; ++b) {
            char* p = X + (size_t)b * plane;
            CK(h, cudaMemcpyAsync(p, p + (size_t)g.H * row, halo, cudaMemcpyDeviceToDevice, st));                    // top halo <- bottom own
            CK(h, cudaMemcpyAsync(p + (size_t)(g.H + 3) * row, p + 3 * row, halo, cudaMemcpyDeviceToDevice, st));    // bottom halo <- top own
        }
        return SLIME_CA_OK;
    }
    const nccl::Api& n = nccl::api();
    nccl::comm_t comm = (nccl::comm_t)h->comm;
    const int up = (h->ring_rank + h->ring_world - 1) % h->ring_world, down = (h->ring_rank + 1) % h->ring_world;
    NK(h, n.GroupStart());
    for (int b = 0; b < g.B; ++b) {
        char* p = X + (size_t)b * plane;
        // Sends and receives between one pair of ranks match in the order they are issued.  Every rank sends "top
        // own rows up" before "bottom own rows down", so with two ranks (up == down) the peer's first message is
        // its top rows, which belong in my bottom halo: receive the bottom halo first.
        NK(h, n.Send(p + 3 * row, halo, nccl::DT_UINT8, up, comm, st));
        NK(h, n.Send(p + (size_t)g.H * row, halo, nccl::DT_UINT8, down, comm, st));
        NK(h, n.Recv(p + (size_t)(g.H + 3) * row, halo, nccl::DT_UINT8, down, comm, st));
        NK(h, n.Recv(p, halo, nccl::DT_UINT8, up, comm, st));
    }
    NK(h, n.GroupEnd());
    return SLIME_CA_OK;
}

int ring_allreduce(slime_ca* h, double* buf, cudaStream_t st) {
    if (h->ring_world == 1) return SLIME_CA_OK;
    const nccl::Api& n = nccl::api();
    NK(h, n.AllReduce(buf, buf, (size_t)h->g.B * NC, nccl::DT_FLOAT64, nccl::OP_SUM, (nccl::comm_t)h->comm, st));
    return SLIME_CA_OK;
}

int ring_ready(slime_ca* h) {
    int rc = ready(h);
    if (rc) return rc;
    if (h->ring_world <= 0) return fail(h, SLIME_CA_ESTATE, "no ring attached: call slime_ca_ring_init or slime_ca_ring_attach first");
    return SLIME_CA_OK;
}

const char* const AFTER_EDEVICE = "); the state is no longer defined: load it again before further steps";

// After a synchronisation: read the device status word itself.
int check_status_word(slime_ca* h) {
    int s = 0;
    CK(h, cudaMemcpy(&s, h->dev_status, sizeof(int), cudaMemcpyDeviceToHost));
    if (s != 0) {
        cudaMemset(h->dev_status, 0, sizeof(int));
        *reinterpret_cast<volatile int*>(h->host_status) = 0;
        return fail(h, SLIME_CA_EDEVICE, "a kernel gave up on a bounded wait (status word " + std::to_string(s) + AFTER_EDEVICE);
    }
    return SLIME_CA_OK;
}

// Without synchronising: the mirror that the last batch of steps copied back, if that copy has run by now.  Lets a
// caller that never leaves the device (set_state_device / step / get_state_device) learn of a failed wait at its
// next call.
int poll_status(slime_ca* h, cudaStream_t st) {
    const int s = *reinterpret_cast<volatile int*>(h->host_status);
    if (s == 0) return SLIME_CA_OK;
    *reinterpret_cast<volatile int*>(h->host_status) = 0;
    cudaMemsetAsync(h->dev_status, 0, sizeof(int), st);
    return fail(h, SLIME_CA_EDEVICE, "a kernel of an earlier call gave up on a bounded wait (status word " + std::to_string(s) + AFTER_EDEVICE);
}

int publish_status(slime_ca* h, cudaStream_t st) {
    CK(h, cudaMemcpyAsync(h->host_status, h->dev_status, sizeof(int), cudaMemcpyDeviceToHost, st));
    return SLIME_CA_OK;
}

}  // namespace

extern "C" {

int slime_ca_create(const slime_ca_config* cfg, slime_ca** out) {
    if (!cfg || !out) return SLIME_CA_EINVAL;
    *out = nullptr;
    if (cfg->batch <= 0 || cfg->height <= 0 || cfg->width <= 0 || cfg->n_weight_sets <= 0 ||
        cfg->batch % cfg->n_weight_sets != 0 || (cfg->dtype != SLIME_CA_F32 && cfg->dtype != SLIME_CA_BF16) ||
        (cfg->stripe != 0 && cfg->stripe != 1))
        return SLIME_CA_EINVAL;
    int ndev = 0;
    if (cudaGetDeviceCount(&ndev) != cudaSuccess || cfg->device < 0 || cfg->device >= ndev) {
        cudaGetLastError();
        return SLIME_CA_ECUDA;
    }
    slime_ca* h = new (std::nothrow) slime_ca();
    if (!h) return SLIME_CA_ENOMEM;
    *out = h;  // returned even on failure so that slime_ca_last_error() can be read; destroy it either way
    h->cfg = *cfg;
    CK(h, cudaSetDevice(cfg->device));
    cudaDeviceProp prop{};
    CK(h, cudaGetDeviceProperties(&prop, cfg->device));
    if (prop.major != 10) return fail(h, SLIME_CA_ECUDA, "this library is built for sm_100a only; device is sm_" +
                                                              std::to_string(prop.major) + std::to_string(prop.minor));
    Geom& g = h->g;
    g.B = cfg->batch; g.H = cfg->height; g.W = cfg->width;
    g.hx = cfg->stripe ? 3 : 0; g.he = cfg->stripe ? 2 : 0;
    g.wrap_y = cfg->stripe ? 0 : 1;
    g.per_set = cfg->batch / cfg->n_weight_sets;
    g.dt = cfg->dt;
    h->esz = cfg->dtype == SLIME_CA_BF16 ? 2 : 4;
    if (cfg->dtype == SLIME_CA_BF16) { g.ev_h = g.H + 2 * APRON; g.ev_w = g.W + 2 * APRON; }
    else { g.ev_h = g.H + 2 * g.he; g.ev_w = g.W; }
    h->weights_set.assign(cfg->n_weight_sets, 0);

    const size_t xn = (size_t)g.B * g.state_rows() * g.W * NC;
    const size_t en = (size_t)g.B * NH * g.ev_h * g.ev_w * HD;
    int rc;
    if (is_bf16(h)) {
        bf16_plan(h->bf, g);
        g.tiles_x = h->bf.tiles_x;
        h->k1_tiles = h->bf.k1_tiles; h->k2_tiles = h->bf.k2_tiles;
    } else {
        g.tiles_x = (g.W + T32 - 1) / T32;
        h->k1_tiles = g.tiles_x * ((g.H + 2 * g.he + T32 - 1) / T32);
        h->k2_tiles = g.tiles_x * ((g.H + T32 - 1) / T32);
        CK(h, cudaFuncSetAttribute(k1_f32, cudaFuncAttributeMaxDynamicSharedMemorySize, K1F32_SMEM));
        CK(h, cudaFuncSetAttribute(k2_f32, cudaFuncAttributeMaxDynamicSharedMemorySize, K2F32_SMEM));
    }
    h->tiles_x = g.tiles_x;
    const int chunks = (int)(((size_t)g.H * g.W + 255) / 256);
    h->partial_cap = h->k2_tiles > chunks ? h->k2_tiles : chunks;

    char* p = nullptr;
    if ((rc = dev_alloc(h, &p, xn * h->esz))) return rc; h->X = p;
    if ((rc = dev_alloc(h, &p, en * h->esz))) return rc; h->E = p;
    if ((rc = dev_alloc(h, &p, en * h->esz))) return rc; h->V = p;
    CK(h, cudaMemset(h->X, 0, xn * h->esz));
    if (cfg->keep_vprime) {
        const size_t vn = (size_t)g.B * NH * g.H * g.W * HD;
        for (int i = 0; i < 2; ++i) { if ((rc = dev_alloc(h, &p, vn * h->esz))) return rc; h->vprime[i] = p; }
        const size_t cells = (size_t)g.H * g.W;
        h->gram_splits = (int)((cells + GRAM_CHUNK - 1) / GRAM_CHUNK);
        if (h->gram_splits > 64) h->gram_splits = 64;   // k_gram then covers GRAM_CHUNK * 64 cells at most
        if ((size_t)h->gram_splits * GRAM_CHUNK < cells)
            return fail(h, SLIME_CA_EINVAL, "keep_vprime supports grids of at most 131072 cells");
        if ((rc = dev_alloc(h, &h->gram_part, (size_t)g.B * NH * h->gram_splits * HD * HD))) return rc;
        if (is_bf16(h))
            for (int i = 0; i < 2; ++i)
                if (gram_tc_map(&h->gram_map[i], h->vprime[i], g.B * NH, (int)cells) != 0)
                    return fail(h, SLIME_CA_ECUDA, "tensor-map set-up of the Gram kernel failed");
        if ((rc = dev_alloc(h, &h->head_rank, (size_t)g.B * NH))) return rc;
        h->pearson_splits = (int)((cells * HC + 262143) / 262144);
        if (h->pearson_splits > 64) h->pearson_splits = 64;
        if ((rc = dev_alloc(h, &h->pearson_part, (size_t)g.B * h->pearson_splits * 5))) return rc;
        if ((rc = dev_alloc(h, &h->fit_dev, (size_t)g.B * 4))) return rc;
    }
    if ((rc = dev_alloc(h, &h->scale, (size_t)g.B * NC))) return rc;
    if ((rc = dev_alloc(h, &h->mass, (size_t)g.B * NC))) return rc;
    if ((rc = dev_alloc(h, &h->sums, (size_t)g.B * NC))) return rc;
    h->partial_lo = is_bf16(h) ? 0 : (size_t)g.B * h->partial_cap * NC;
    if ((rc = dev_alloc(h, &h->partial, (size_t)g.B * h->partial_cap * NC + h->partial_lo))) return rc;
    if ((rc = dev_alloc(h, &h->seg_sums, (size_t)g.B * 64 * NC))) return rc;
    if ((rc = dev_alloc(h, &h->tickets, (size_t)g.B))) return rc;
    CK(h, cudaMemset(h->tickets, 0, (size_t)g.B * sizeof(int)));
    if ((rc = dev_alloc(h, &h->dev_status, 1))) return rc;
    CK(h, cudaMemset(h->dev_status, 0, sizeof(int)));
    CK(h, cudaHostAlloc((void**)&h->host_status, sizeof(int), cudaHostAllocDefault));
    *h->host_status = 0;
    const size_t sets = cfg->n_weight_sets;
    if ((rc = dev_alloc(h, &h->prm, sets * NH * PRM))) return rc;
    if ((rc = dev_alloc(h, &h->master, sets * MW_STRIDE))) return rc;
    CK(h, cudaMemset(h->master, 0, sets * MW_STRIDE * sizeof(float)));
    if ((rc = dev_alloc(h, &h->set_stats, sets * 2))) return rc;
    if ((rc = dev_alloc(h, &h->parent, sets))) return rc;
    if ((rc = dev_alloc(h, &h->evolve_info, 2))) return rc;
    if (is_bf16(h)) {
        if ((rc = dev_alloc(h, &h->w1_bf16, sets * NH * 192 * 64))) return rc;
        if ((rc = dev_alloc(h, &h->wo_bf16, sets * NH * 64 * 64))) return rc;
        if (bf16_setup(h->bf, h->w1_bf16, h->wo_bf16, (int)sets, (const __nv_bfloat16*)h->E, (const __nv_bfloat16*)h->V,
                       (const __nv_bfloat16*)h->X, g,
                       prop.multiProcessorCount) != 0)
            return fail(h, SLIME_CA_ECUDA, "tensor-map / kernel attribute set-up failed: " + std::string(bf16_error()));
    } else {
        if ((rc = dev_alloc(h, &h->wpiv_f32, sets * NH * NC * 192))) return rc;
        if ((rc = dev_alloc(h, &h->wo_f32, sets * NH * HD * NC))) return rc;
    }
    std::vector<float> ones((size_t)g.B * NC, 1.f);
    CK(h, cudaMemcpy(h->scale, ones.data(), ones.size() * sizeof(float), cudaMemcpyHostToDevice));
    return SLIME_CA_OK;
}

int slime_ca_destroy(slime_ca* h) {
    if (!h) return SLIME_CA_EINVAL;
    cudaSetDevice(h->cfg.device);
    void* ptrs[] = {h->X, h->E, h->V, h->vprime[0], h->vprime[1], h->scale, h->mass, h->sums, h->partial, h->seg_sums, h->tickets,
                    h->wpiv_f32, h->wo_f32, h->prm, h->w1_bf16, h->wo_bf16, h->gram_part, h->head_rank,
                    h->pearson_part, h->fit_dev, h->dev_status, h->master, h->set_stats, h->parent, h->evolve_info};
    for (void* p : ptrs)
        if (p) cudaFree(p);
    if (h->host_status) cudaFreeHost(h->host_status);
    ring_release(h);
    delete h;
    return SLIME_CA_OK;
}

const char* slime_ca_last_error(const slime_ca* h) { return h ? h->err.c_str() : "null handle"; }
size_t slime_ca_workspace_bytes(const slime_ca* h) { return h ? h->bytes : 0; }
long long slime_ca_launch_count(const slime_ca* h) { return h ? h->launches : 0; }

int slime_ca_set_weights(slime_ca* h, int set_index, const float* Wp, const float* Wi, const float* Wv,
                         const float* Wo, const float* K, const float* mu, const float* sigma) {
    if (!h) return SLIME_CA_EINVAL;
    if (!Wp || !Wi || !Wv || !Wo || !K || !mu || !sigma) return fail(h, SLIME_CA_EINVAL, "null weight pointer");
    if (set_index < 0 || set_index >= h->cfg.n_weight_sets) return fail(h, SLIME_CA_EINVAL, "weight set index out of range");
    for (int i = 0; i < NH; ++i)
        if (!(sigma[i] > 0.f)) return fail(h, SLIME_CA_EINVAL, "sigma must be positive");
    CK(h, cudaSetDevice(h->cfg.device));
    // Steps still in flight on any stream (non-blocking streams are not ordered against the copies below) read the
    // arrays this call overwrites: wait for the device to drain first.
    CK(h, cudaDeviceSynchronize());
    // The fp32 master copy stays on the device (the population step mutates it there); the operand layouts of
    // the step kernels are derived from it by a kernel.
    float* m = h->master + (size_t)set_index * MW_STRIDE;
    CK(h, cudaMemcpy(m + MW_WP, Wp, (size_t)NH * NC * HD * sizeof(float), cudaMemcpyHostToDevice));
    CK(h, cudaMemcpy(m + MW_WI, Wi, (size_t)NH * NC * HD * sizeof(float), cudaMemcpyHostToDevice));
    CK(h, cudaMemcpy(m + MW_WV, Wv, (size_t)NH * NC * HD * sizeof(float), cudaMemcpyHostToDevice));
    CK(h, cudaMemcpy(m + MW_WO, Wo, (size_t)NH * HD * NC * sizeof(float), cudaMemcpyHostToDevice));
    CK(h, cudaMemcpy(m + MW_K, K, NH * 9 * sizeof(float), cudaMemcpyHostToDevice));
    CK(h, cudaMemcpy(m + MW_MU, mu, NH * sizeof(float), cudaMemcpyHostToDevice));
    CK(h, cudaMemcpy(m + MW_SIGMA, sigma, NH * sizeof(float), cudaMemcpyHostToDevice));
    k_weights_layout<<<dim3(32, 1), 256>>>(h->master, nullptr, set_index, is_bf16(h) ? 1 : 0, h->wpiv_f32, h->wo_f32,
                                           h->w1_bf16, h->wo_bf16, h->prm);
    LAUNCHED(h);
    CK(h, cudaStreamSynchronize(nullptr));
    h->weights_set[set_index] = 1;
    return SLIME_CA_OK;
}

int slime_ca_set_state_device(slime_ca* h, const void* dev_state, int dtype, void* stream) {
    if (!h) return SLIME_CA_EINVAL;
    if (!dev_state || (dtype != SLIME_CA_F32 && dtype != SLIME_CA_BF16)) return fail(h, SLIME_CA_EINVAL, "bad state pointer or dtype");
    CK(h, cudaSetDevice(h->cfg.device));
    cudaStream_t st = (cudaStream_t)stream;
    {
        const int bad = *reinterpret_cast<volatile int*>(h->host_status);   // a fresh state ends an earlier failure
        if (bad) { *reinterpret_cast<volatile int*>(h->host_status) = 0; cudaMemsetAsync(h->dev_status, 0, sizeof(int), st); }
    }
    const Geom& g = h->g;
    const size_t n = (size_t)g.B * g.H * g.W * NC;
    const int blocks = grid_for(n);
    if (is_bf16(h)) {
        if (dtype == SLIME_CA_BF16) k_state_in<__nv_bfloat16, __nv_bfloat16><<<blocks, 256, 0, st>>>((const __nv_bfloat16*)dev_state, (__nv_bfloat16*)h->X, g);
        else k_state_in<float, __nv_bfloat16><<<blocks, 256, 0, st>>>((const float*)dev_state, (__nv_bfloat16*)h->X, g);
    } else {
        if (dtype == SLIME_CA_BF16) k_state_in<__nv_bfloat16, float><<<blocks, 256, 0, st>>>((const __nv_bfloat16*)dev_state, (float*)h->X, g);
        else k_state_in<float, float><<<blocks, 256, 0, st>>>((const float*)dev_state, (float*)h->X, g);
    }
    LAUNCHED(h);
    int rc = channel_sums(h, 1, st);
    if (rc) return rc;
    h->state_set = true;
    h->vp_steps = 0; h->fitness_valid = false;
    return SLIME_CA_OK;
}

int slime_ca_get_state_device(slime_ca* h, void* dev_state, int dtype, void* stream) {
    if (!h) return SLIME_CA_EINVAL;
    if (!dev_state || (dtype != SLIME_CA_F32 && dtype != SLIME_CA_BF16)) return fail(h, SLIME_CA_EINVAL, "bad state pointer or dtype");
    if (!h->state_set) return fail(h, SLIME_CA_ESTATE, "no state has been loaded");
    CK(h, cudaSetDevice(h->cfg.device));
    cudaStream_t st = (cudaStream_t)stream;
    int rcs = poll_status(h, st);
    if (rcs) return rcs;
    const Geom& g = h->g;
    const int blocks = grid_for((size_t)g.B * g.H * g.W * NC);
    if (is_bf16(h)) {
        if (dtype == SLIME_CA_BF16) k_state_out<__nv_bfloat16, __nv_bfloat16><<<blocks, 256, 0, st>>>((const __nv_bfloat16*)h->X, h->scale, (__nv_bfloat16*)dev_state, g);
        else k_state_out<__nv_bfloat16, float><<<blocks, 256, 0, st>>>((const __nv_bfloat16*)h->X, h->scale, (float*)dev_state, g);
    } else {
        if (dtype == SLIME_CA_BF16) k_state_out<float, __nv_bfloat16><<<blocks, 256, 0, st>>>((const float*)h->X, h->scale, (__nv_bfloat16*)dev_state, g);
        else k_state_out<float, float><<<blocks, 256, 0, st>>>((const float*)h->X, h->scale, (float*)dev_state, g);
    }
    LAUNCHED(h);
    return SLIME_CA_OK;
}

// Host transfers stage through the E intermediate (always at least 8x the state), so no extra memory.
int slime_ca_set_state(slime_ca* h, const void* host_state, int host_dtype, void* stream) {
    if (!h) return SLIME_CA_EINVAL;
    if (!host_state || (host_dtype != SLIME_CA_F32 && host_dtype != SLIME_CA_BF16)) return fail(h, SLIME_CA_EINVAL, "bad state pointer or dtype");
    CK(h, cudaSetDevice(h->cfg.device));
    cudaStream_t st = (cudaStream_t)stream;
    const size_t n = (size_t)h->g.B * h->g.H * h->g.W * NC;
    CK(h, cudaMemcpyAsync(h->E, host_state, n * (host_dtype == SLIME_CA_BF16 ? 2 : 4), cudaMemcpyHostToDevice, st));
    int rc = slime_ca_set_state_device(h, h->E, host_dtype, stream);
    if (rc) return rc;
    CK(h, cudaStreamSynchronize(st));
    return SLIME_CA_OK;
}

int slime_ca_get_state(slime_ca* h, void* host_state, int host_dtype, void* stream) {
    if (!h) return SLIME_CA_EINVAL;
    if (!host_state) return fail(h, SLIME_CA_EINVAL, "null state pointer");
    int rc = slime_ca_get_state_device(h, h->E, host_dtype, stream);
    if (rc) return rc;
    cudaStream_t st = (cudaStream_t)stream;
    const size_t n = (size_t)h->g.B * h->g.H * h->g.W * NC;
    CK(h, cudaMemcpyAsync(host_state, h->E, n * (host_dtype == SLIME_CA_BF16 ? 2 : 4), cudaMemcpyDeviceToHost, st));
    CK(h, cudaStreamSynchronize(st));
    return check_status_word(h);
}

int slime_ca_set_mass(slime_ca* h, const double* mass) {
    if (!h) return SLIME_CA_EINVAL;
    if (!mass) return fail(h, SLIME_CA_EINVAL, "null mass pointer");
    CK(h, cudaSetDevice(h->cfg.device));
    CK(h, cudaMemcpy(h->mass, mass, (size_t)h->g.B * NC * sizeof(double), cudaMemcpyHostToDevice));
    return SLIME_CA_OK;
}

int slime_ca_get_mass(slime_ca* h, double* mass) {
    if (!h) return SLIME_CA_EINVAL;
    if (!mass) return fail(h, SLIME_CA_EINVAL, "null mass pointer");
    CK(h, cudaSetDevice(h->cfg.device));
    CK(h, cudaMemcpy(mass, h->mass, (size_t)h->g.B * NC * sizeof(double), cudaMemcpyDeviceToHost));
    return SLIME_CA_OK;
}

int slime_ca_step_partial(slime_ca* h, void* stream) {
    int rc = ready(h);
    if (rc) return rc;
    CK(h, cudaSetDevice(h->cfg.device));
    if ((rc = poll_status(h, (cudaStream_t)stream))) return rc;
    void* emit = nullptr;
    if (h->cfg.keep_vprime) { h->vp_last ^= 1; emit = h->vprime[h->vp_last]; ++h->vp_steps; h->fitness_valid = false; }
    rc = step_kernels(h, emit, (cudaStream_t)stream);
    if (rc) return rc;
    ++h->steps_done;
    return publish_status(h, (cudaStream_t)stream);
}

int slime_ca_step_finish(slime_ca* h, void* stream) {
    int rc = ready(h);
    if (rc) return rc;
    CK(h, cudaSetDevice(h->cfg.device));
    const int n = h->g.B * NC;
    k_scale_from_sums<<<(n + 255) / 256, 256, 0, (cudaStream_t)stream>>>(h->sums, h->mass, h->scale, n);
    LAUNCHED(h);
    return SLIME_CA_OK;
}

int slime_ca_step(slime_ca* h, int n_steps, void* stream) {
    int rc = ready(h);
    if (rc) return rc;
    if (n_steps < 0) return fail(h, SLIME_CA_EINVAL, "negative step count");
    CK(h, cudaSetDevice(h->cfg.device));
    cudaStream_t st = (cudaStream_t)stream;
    if ((rc = poll_status(h, st))) return rc;
    for (int i = 0; i < n_steps; ++i) {
        void* emit = nullptr;
        if (h->cfg.keep_vprime && i >= n_steps - 2) { h->vp_last ^= 1; emit = h->vprime[h->vp_last]; ++h->vp_steps; h->fitness_valid = false; }
        rc = step_kernels(h, emit, st, nullptr, 2);
        if (rc) return rc;
        ++h->steps_done;
    }
    return n_steps > 0 ? publish_status(h, st) : SLIME_CA_OK;
}

int slime_ca_step_timed(slime_ca* h, int n_steps, void* stream, float* ms) {
    int rc = ready(h);
    if (rc) return rc;
    if (n_steps <= 0 || n_steps > 4096 || !ms) return fail(h, SLIME_CA_EINVAL, "bad step count or null output");
    CK(h, cudaSetDevice(h->cfg.device));
    cudaStream_t st = (cudaStream_t)stream;
    struct Events {          // destroyed on every way out of this function
        std::vector<cudaEvent_t> v;
        ~Events() { for (cudaEvent_t e : v) if (e) cudaEventDestroy(e); }
    } evs;
    evs.v.assign((size_t)n_steps * 4, nullptr);
    std::vector<cudaEvent_t>& ev = evs.v;
    for (auto& e : ev) CK(h, cudaEventCreate(&e));
    h->vp_steps = 0; h->fitness_valid = false;      // these steps do not emit V': the kept pair no longer matches the state
    for (int i = 0; i < n_steps; ++i) {
        rc = step_kernels(h, nullptr, st, &ev[(size_t)i * 4], 2);
        if (rc) return rc;
        CK(h, cudaEventRecord(ev[(size_t)i * 4 + 3], st));
        ++h->steps_done;
    }
    CK(h, cudaStreamSynchronize(st));
    ms[0] = ms[1] = ms[2] = 0.f;
    for (int i = 0; i < n_steps; ++i)
        for (int k = 0; k < 3; ++k) {
            float t = 0.f;
            CK(h, cudaEventElapsedTime(&t, ev[(size_t)i * 4 + k], ev[(size_t)i * 4 + k + 1]));
            ms[k] += t;
        }
    return check_status_word(h);
}

int slime_ca_buffer(slime_ca* h, int which, void** dev_ptr, size_t* bytes) {
    if (!h) return SLIME_CA_EINVAL;
    if (!dev_ptr || !bytes) return fail(h, SLIME_CA_EINVAL, "null output pointer");
    const Geom& g = h->g;
    const size_t vn = (size_t)g.B * NH * g.H * g.W * HD * h->esz;
    switch (which) {
        case SLIME_CA_BUF_STATE: *dev_ptr = h->X; *bytes = (size_t)g.B * g.state_rows() * g.W * NC * h->esz; break;
        case SLIME_CA_BUF_SCALE: *dev_ptr = h->scale; *bytes = (size_t)g.B * NC * sizeof(float); break;
        case SLIME_CA_BUF_MASS: *dev_ptr = h->mass; *bytes = (size_t)g.B * NC * sizeof(double); break;
        case SLIME_CA_BUF_SUMS: *dev_ptr = h->sums; *bytes = (size_t)g.B * NC * sizeof(double); break;
        case SLIME_CA_BUF_VPRIME_PREV: *dev_ptr = h->vprime[h->vp_last ^ 1]; *bytes = h->vprime[0] ? vn : 0; break;
        case SLIME_CA_BUF_VPRIME_LAST: *dev_ptr = h->vprime[h->vp_last]; *bytes = h->vprime[0] ? vn : 0; break;
        default: return fail(h, SLIME_CA_EINVAL, "unknown buffer id");
    }
    return SLIME_CA_OK;
}

int slime_ca_fitness(slime_ca* h, float* rank, float* coherence, float* fitness, float* hunger, void* stream) {
    int rc = ready(h);
    if (rc) return rc;
    if (!h->cfg.keep_vprime) return fail(h, SLIME_CA_ESTATE, "handle was created without keep_vprime");
    if (h->vp_steps < 2) return fail(h, SLIME_CA_ESTATE, "fitness needs two steps since the state was loaded");
    CK(h, cudaSetDevice(h->cfg.device));
    cudaStream_t st = (cudaStream_t)stream;
    const Geom& g = h->g;
    const int cells = g.H * g.W;
    const void* va = h->vprime[h->vp_last ^ 1];
    const void* vb = h->vprime[h->vp_last];
    const size_t per_grid = (size_t)cells * HC;
    if (is_bf16(h)) {
        k_gram_tc<<<g.B * NH, 128, gtc::SMEM, st>>>(h->gram_map[h->vp_last], cells, h->gram_splits, h->gram_part, h->dev_status);
        LAUNCHED(h);
        k_pearson<__nv_bfloat16><<<dim3(h->pearson_splits, g.B), 256, 0, st>>>((const __nv_bfloat16*)va, (const __nv_bfloat16*)vb, per_grid, h->pearson_part);
        LAUNCHED(h);
    } else {
        k_gram<float><<<dim3(h->gram_splits, NH, g.B), GRAM_THREADS, 0, st>>>((const float*)vb, cells, h->gram_part);
        LAUNCHED(h);
        k_pearson<float><<<dim3(h->pearson_splits, g.B), 256, 0, st>>>((const float*)va, (const float*)vb, per_grid, h->pearson_part);
        LAUNCHED(h);
    }
    k_jacobi_rank<<<g.B * NH, JACOBI_THREADS, 0, st>>>(h->gram_part, h->gram_splits, h->head_rank);
    LAUNCHED(h);
    k_fitness_final<<<(g.B + 127) / 128, 128, 0, st>>>(h->head_rank, h->pearson_part, h->pearson_splits, (double)per_grid, h->fit_dev, g.B);
    LAUNCHED(h);
    std::vector<float> out((size_t)g.B * 4);
    CK(h, cudaMemcpyAsync(out.data(), h->fit_dev, out.size() * sizeof(float), cudaMemcpyDeviceToHost, st));
    CK(h, cudaStreamSynchronize(st));
    for (int b = 0; b < g.B; ++b) {
        if (rank) rank[b] = out[b * 4 + 0];
        if (coherence) coherence[b] = out[b * 4 + 1];
        if (fitness) fitness[b] = out[b * 4 + 2];
        if (hunger) hunger[b] = out[b * 4 + 3];
    }
    h->fitness_valid = true;
    return check_status_word(h);
}

int slime_ca_get_weights(slime_ca* h, int set_index, float* Wp, float* Wi, float* Wv, float* Wo, float* K, float* mu,
                         float* sigma) {
    if (!h) return SLIME_CA_EINVAL;
    if (set_index < 0 || set_index >= h->cfg.n_weight_sets) return fail(h, SLIME_CA_EINVAL, "weight set index out of range");
    if (!h->weights_set[set_index]) return fail(h, SLIME_CA_ESTATE, "this weight set has not been uploaded");
    CK(h, cudaSetDevice(h->cfg.device));
    const float* m = h->master + (size_t)set_index * MW_STRIDE;
    const size_t nm = (size_t)NH * NC * HD * sizeof(float);
    if (Wp) CK(h, cudaMemcpy(Wp, m + MW_WP, nm, cudaMemcpyDeviceToHost));
    if (Wi) CK(h, cudaMemcpy(Wi, m + MW_WI, nm, cudaMemcpyDeviceToHost));
    if (Wv) CK(h, cudaMemcpy(Wv, m + MW_WV, nm, cudaMemcpyDeviceToHost));
    if (Wo) CK(h, cudaMemcpy(Wo, m + MW_WO, nm, cudaMemcpyDeviceToHost));
    if (K) CK(h, cudaMemcpy(K, m + MW_K, NH * 9 * sizeof(float), cudaMemcpyDeviceToHost));
    if (mu) CK(h, cudaMemcpy(mu, m + MW_MU, NH * sizeof(float), cudaMemcpyDeviceToHost));
    if (sigma) CK(h, cudaMemcpy(sigma, m + MW_SIGMA, NH * sizeof(float), cudaMemcpyDeviceToHost));
    return SLIME_CA_OK;
}

int slime_ca_evolve(slime_ca* h, const slime_ca_evolve_params* p, int* parent, int* best_set, int* n_replaced,
                    void* stream) {
    int rc = ready(h);
    if (rc) return rc;
    if (!p) return fail(h, SLIME_CA_EINVAL, "null parameters");
    if (!(p->mutation_rate >= 0.f && p->mutation_rate <= 1.f) || !(p->mutation_sigma >= 0.f))
        return fail(h, SLIME_CA_EINVAL, "mutation_rate must lie in [0, 1] and mutation_sigma must not be negative");
    if (!h->cfg.keep_vprime || !h->fitness_valid)
        return fail(h, SLIME_CA_ESTATE, "the population step follows slime_ca_fitness on the same state");
    CK(h, cudaSetDevice(h->cfg.device));
    cudaStream_t st = (cudaStream_t)stream;
    const int sets = h->cfg.n_weight_sets;
    EvolveParams ep{p->fitness_threshold, p->hunger_threshold, p->mutation_rate, p->mutation_sigma, p->seed, p->generation};
    k_evolve_select<<<1, 256, 0, st>>>(h->fit_dev, sets, h->g.per_set, ep, h->set_stats, h->parent, h->evolve_info);
    LAUNCHED(h);
    k_evolve_refill<<<dim3(32, sets), 256, 0, st>>>(h->master, h->parent, ep);
    LAUNCHED(h);
    k_weights_layout<<<dim3(32, sets), 256, 0, st>>>(h->master, h->parent, 0, is_bf16(h) ? 1 : 0, h->wpiv_f32, h->wo_f32,
                                                     h->w1_bf16, h->wo_bf16, h->prm);
    LAUNCHED(h);
    int info[2] = {-1, 0};
    CK(h, cudaMemcpyAsync(info, h->evolve_info, sizeof(info), cudaMemcpyDeviceToHost, st));
    if (parent) CK(h, cudaMemcpyAsync(parent, h->parent, sets * sizeof(int), cudaMemcpyDeviceToHost, st));
    CK(h, cudaStreamSynchronize(st));
    h->evolved = true;
    if (best_set) *best_set = info[0];
    if (n_replaced) *n_replaced = info[1];
    return SLIME_CA_OK;
}

int slime_ca_lift_images(slime_ca* h, const float* host_img, int img_h, int img_w, const float* host_L, void* stream) {
    if (!h) return SLIME_CA_EINVAL;
    if (!host_img || !host_L || img_h <= 0 || img_w <= 0 || img_h > h->g.H || img_w > h->g.W)
        return fail(h, SLIME_CA_EINVAL, "bad image pointer or image larger than the grid");
    CK(h, cudaSetDevice(h->cfg.device));
    cudaStream_t st = (cudaStream_t)stream;
    const Geom& g = h->g;
    const size_t n_img = (size_t)g.B * img_h * img_w;
    float* d_img = (float*)h->E;
    float* d_L = (float*)h->V;
    CK(h, cudaMemcpyAsync(d_img, host_img, n_img * sizeof(float), cudaMemcpyHostToDevice, st));
    CK(h, cudaMemcpyAsync(d_L, host_L, NC * sizeof(float), cudaMemcpyHostToDevice, st));
    const int blocks = grid_for((size_t)g.B * g.H * g.W * NC);
    if (is_bf16(h)) k_lift<__nv_bfloat16><<<blocks, 256, 0, st>>>(d_img, img_h, img_w, d_L, (__nv_bfloat16*)h->X, g);
    else k_lift<float><<<blocks, 256, 0, st>>>(d_img, img_h, img_w, d_L, (float*)h->X, g);
    LAUNCHED(h);
    int rc = channel_sums(h, 1, st);
    if (rc) return rc;
    CK(h, cudaStreamSynchronize(st));
    h->state_set = true;
    h->vp_steps = 0; h->fitness_valid = false;
    return SLIME_CA_OK;
}

int slime_ca_pool_readout(slime_ca* h, const float* host_Wr, const float* host_br, int n_out, float* host_logits, void* stream) {
    if (!h) return SLIME_CA_EINVAL;
    if (!host_Wr || !host_logits || n_out <= 0 || n_out > 1024) return fail(h, SLIME_CA_EINVAL, "bad readout arguments");
    if (!h->state_set) return fail(h, SLIME_CA_ESTATE, "no state has been loaded");
    {
        // Wr, br and the logits are staged in the E intermediate (free between steps): they have to fit there
        const Geom& g0 = h->g;
        const size_t need = ((size_t)NC * n_out + n_out + (size_t)g0.B * n_out) * sizeof(float);
        const size_t have = (size_t)g0.B * NH * g0.ev_h * g0.ev_w * HD * h->esz;
        if (need > have)
            return fail(h, SLIME_CA_EINVAL, "read-out too wide for this handle: (64 * n_out + n_out + batch * n_out) * 4 = " +
                                                std::to_string(need) + " bytes exceed the " + std::to_string(have) +
                                                "-byte staging buffer (batch * 8 * rows * columns * 64 elements)");
    }
    CK(h, cudaSetDevice(h->cfg.device));
    cudaStream_t st = (cudaStream_t)stream;
    const Geom& g = h->g;
    int rc = channel_sums(h, 0, st);   // sums of what is stored now; mass and scale untouched
    if (rc) return rc;
    float* d_W = (float*)h->E;
    float* d_b = d_W + (size_t)NC * n_out;
    float* d_out = d_b + n_out;
    CK(h, cudaMemcpyAsync(d_W, host_Wr, (size_t)NC * n_out * sizeof(float), cudaMemcpyHostToDevice, st));
    if (host_br) CK(h, cudaMemcpyAsync(d_b, host_br, n_out * sizeof(float), cudaMemcpyHostToDevice, st));
    k_pool_readout<<<g.B, ((n_out + 31) / 32) * 32, 0, st>>>(h->sums, h->scale, 1.0 / ((double)g.H * g.W), d_W, host_br ? d_b : nullptr, n_out, d_out);
    LAUNCHED(h);
    CK(h, cudaMemcpyAsync(host_logits, d_out, (size_t)g.B * n_out * sizeof(float), cudaMemcpyDeviceToHost, st));
    CK(h, cudaStreamSynchronize(st));
    return SLIME_CA_OK;
}

int slime_ca_lift_field_device(slime_ca* h, const float* dev_field, const float* host_L, void* stream) {
    if (!h) return SLIME_CA_EINVAL;
    if (!dev_field || !host_L) return fail(h, SLIME_CA_EINVAL, "null field or lift vector");
    CK(h, cudaSetDevice(h->cfg.device));
    cudaStream_t st = (cudaStream_t)stream;
    const Geom& g = h->g;
    float* d_L = (float*)h->V;
    CK(h, cudaMemcpyAsync(d_L, host_L, NC * sizeof(float), cudaMemcpyHostToDevice, st));
    const int blocks = grid_for((size_t)g.B * g.H * g.W * NC);
    if (is_bf16(h)) k_lift<__nv_bfloat16><<<blocks, 256, 0, st>>>(dev_field, g.H, g.W, d_L, (__nv_bfloat16*)h->X, g);
    else k_lift<float><<<blocks, 256, 0, st>>>(dev_field, g.H, g.W, d_L, (float*)h->X, g);
    LAUNCHED(h);
    int rc = channel_sums(h, 1, st);
    if (rc) return rc;
    CK(h, cudaStreamSynchronize(st));
    h->state_set = true;
    h->vp_steps = 0; h->fitness_valid = false;
    return SLIME_CA_OK;
}

int slime_ca_field_from_state_device(slime_ca* h, float* dev_field, void* stream) {
    if (!h) return SLIME_CA_EINVAL;
    if (!dev_field) return fail(h, SLIME_CA_EINVAL, "null field");
    if (!h->state_set) return fail(h, SLIME_CA_ESTATE, "no state has been loaded");
    CK(h, cudaSetDevice(h->cfg.device));
    cudaStream_t st = (cudaStream_t)stream;
    const Geom& g = h->g;
    const int blocks = grid_for((size_t)g.B * g.H * g.W * 8);
    if (is_bf16(h)) k_channel_mean<__nv_bfloat16><<<blocks, 256, 0, st>>>((const __nv_bfloat16*)h->X, h->scale, dev_field, g);
    else k_channel_mean<float><<<blocks, 256, 0, st>>>((const float*)h->X, h->scale, dev_field, g);
    LAUNCHED(h);
    return SLIME_CA_OK;
}

int slime_ca_set_weights_reference_layout(slime_ca* h, int set_index, const float* dev_perception,
                                          const float* dev_interaction, const float* dev_value,
                                          const float* dev_head_mixing, const float* dev_flow_kernels,
                                          const float* mu, const float* sigma) {
    if (!h) return SLIME_CA_EINVAL;
    if (!dev_perception || !dev_interaction || !dev_value || !dev_head_mixing || !dev_flow_kernels)
        return fail(h, SLIME_CA_EINVAL, "null weight pointer");
    CK(h, cudaSetDevice(h->cfg.device));
    // Only the slices the reference's kernels index are fetched: rows c < 64, columns d < 64 of each head's
    // [512][256] perception / interaction matrix, and columns d < 64 of all 256 rows of the [256][512] value matrix.
    std::vector<float> Wp((size_t)NH * NC * HD), Wi(Wp.size()), Wv(Wp.size()), Wo((size_t)NH * HD * NC, 0.f);
    std::vector<float> val((size_t)256 * HD), mix(NH * NH), K(NH * 9), mu_d(NH, 0.2f), sg_d(NH, 0.03f);
    for (int hd = 0; hd < NH; ++hd) {
        CK(h, cudaMemcpy2D(&Wp[(size_t)hd * NC * HD], HD * sizeof(float), dev_perception + (size_t)hd * 512 * 256,
                           256 * sizeof(float), HD * sizeof(float), NC, cudaMemcpyDeviceToHost));
        CK(h, cudaMemcpy2D(&Wi[(size_t)hd * NC * HD], HD * sizeof(float), dev_interaction + (size_t)hd * 512 * 256,
                           256 * sizeof(float), HD * sizeof(float), NC, cudaMemcpyDeviceToHost));
        CK(h, cudaMemcpy2D(val.data(), HD * sizeof(float), dev_value + (size_t)hd * 256 * 512, 512 * sizeof(float),
                           HD * sizeof(float), 256, cudaMemcpyDeviceToHost));
        for (int c = 0; c < NC; ++c)
            for (int d = 0; d < HD; ++d) {
                float acc = 0.f;     // the reference reads value row j with interaction[j % 64], j < 256
                for (int r = 0; r < 4; ++r) acc += val[(size_t)(c + 64 * r) * HD + d];
                Wv[((size_t)hd * NC + c) * HD + d] = acc;
            }
    }
    CK(h, cudaMemcpy(mix.data(), dev_head_mixing, mix.size() * sizeof(float), cudaMemcpyDeviceToHost));
    CK(h, cudaMemcpy(K.data(), dev_flow_kernels, K.size() * sizeof(float), cudaMemcpyDeviceToHost));
    for (int hd = 0; hd < NH; ++hd) {
        double m = 0.0;              // head mixing followed by the mean of the 8 output heads
        for (int o = 0; o < NH; ++o) m += (double)mix[o * NH + hd];
        for (int d = 0; d < HD; ++d) Wo[((size_t)hd * HD + d) * NC + d] = (float)(m / NH);
    }
    return slime_ca_set_weights(h, set_index, Wp.data(), Wi.data(), Wv.data(), Wo.data(), K.data(),
                                mu ? mu : mu_d.data(), sigma ? sigma : sg_d.data());
}

int slime_ca_evolution_record(slime_ca* h, int grid_index, int generation, double elapsed_seconds,
                              const float* dev_field, int pool_active, int pool_capacity, int pool_spawned,
                              int pool_culled, char* buf, size_t cap, size_t* written, void* stream) {
    if (!h) return SLIME_CA_EINVAL;
    if (!buf || cap == 0 || grid_index < 0 || grid_index >= h->g.B) return fail(h, SLIME_CA_EINVAL, "bad record arguments");
    if (!h->state_set && !dev_field) return fail(h, SLIME_CA_ESTATE, "no state has been loaded");
    CK(h, cudaSetDevice(h->cfg.device));
    cudaStream_t st = (cudaStream_t)stream;
    const Geom& g = h->g;
    const int set = grid_index / g.per_set;
    if (!h->weights_set[set]) return fail(h, SLIME_CA_ESTATE, "this grid's weight set has not been uploaded");
    // the field: the caller's, or the channel mean of the CA state (scratch: the E buffer, free between steps)
    const float* field = dev_field;
    if (!field) {
        float* scratch = (float*)h->E;
        const int blocks = grid_for((size_t)g.B * g.H * g.W * 8);
        if (is_bf16(h)) k_channel_mean<__nv_bfloat16><<<blocks, 256, 0, st>>>((const __nv_bfloat16*)h->X, h->scale, scratch, g);
        else k_channel_mean<float><<<blocks, 256, 0, st>>>((const float*)h->X, h->scale, scratch, g);
        LAUNCHED(h);
        field = scratch + (size_t)grid_index * g.H * g.W;
    }
    const int sh = g.H < 16 ? g.H : 16, sw = g.W < 16 ? g.W : 16;       // centre sample, 16 x 16 on the reference's grid
    const int oy = (g.H - sh) / 2, ox = (g.W - sw) / 2;
    std::vector<float> sample((size_t)sh * sw), taps(NH * 9);
    CK(h, cudaMemcpy2DAsync(sample.data(), sw * sizeof(float), field + (size_t)oy * g.W + ox, g.W * sizeof(float),
                            sw * sizeof(float), sh, cudaMemcpyDeviceToHost, st));
    CK(h, cudaMemcpyAsync(taps.data(), h->master + (size_t)set * MW_STRIDE + MW_K, taps.size() * sizeof(float),
                          cudaMemcpyDeviceToHost, st));
    CK(h, cudaStreamSynchronize(st));
    std::string out;
    char tmp[96];
    auto put = [&](const char* fmt, auto... a) { snprintf(tmp, sizeof(tmp), fmt, a...); out += tmp; };
    put("{\"gen\":%d,\"elapsed\":%.2f,", generation, elapsed_seconds);
    out += "\"chemical\":{\"concentration\":[";
    for (size_t i = 0; i < sample.size(); ++i) { put("%.4f", sample[i]); if (i + 1 < sample.size()) out += ","; }
    put("],\"size\":%d},", sh < sw ? sh : sw);
    out += "\"ca\":{\"flow_kernels\":[";
    for (int hd = 0; hd < NH; ++hd) {
        out += "[";
        for (int t = 0; t < 9; ++t) { put("%.4f", taps[hd * 9 + t]); if (t < 8) out += ","; }
        out += hd + 1 < NH ? "]," : "]";
    }
    out += "]},\"agents\":[],\"voronoi\":[],\"archive\":{\"size\":0,\"elites\":[]},";
    put("\"pool\":{\"active\":%d,\"capacity\":%d,\"spawned\":%d,\"culled\":%d}", pool_active, pool_capacity,
        pool_spawned, pool_culled);
    out += "}\n";
    if (written) *written = out.size();
    if (out.size() + 1 > cap) return fail(h, SLIME_CA_EINVAL, "record needs " + std::to_string(out.size() + 1) + " bytes");
    memcpy(buf, out.c_str(), out.size() + 1);
    return SLIME_CA_OK;
}

void launch_multi_head_ca(float* ca_state, float* weights, float* ca_output, int batch_size, int grid_size) {
    static slime_ca* cached = nullptr;
    if (!ca_state || !weights || !ca_output || batch_size <= 0 || grid_size <= 0) {
        fprintf(stderr, "launch_multi_head_ca: bad arguments\n");
        return;
    }
    int dev = 0;
    cudaGetDevice(&dev);
    if (cached && (cached->cfg.batch != batch_size || cached->cfg.height != grid_size || cached->cfg.device != dev)) {
        slime_ca_destroy(cached);
        cached = nullptr;
    }
    if (!cached) {
        slime_ca_config cfg{batch_size, grid_size, grid_size, 1, SLIME_CA_F32, 0.1f, dev, 0, 1};
        if (slime_ca_create(&cfg, &cached) != SLIME_CA_OK) {
            fprintf(stderr, "launch_multi_head_ca: %s\n", slime_ca_last_error(cached));
            if (cached) slime_ca_destroy(cached);
            cached = nullptr;
            return;
        }
    }
    const size_t wn = (size_t)NH * NC * HD;
    std::vector<float> w(3 * wn), wo((size_t)HC * NC, 0.f), k(NH * 9, 1.f / 9.f), mu(NH, 0.2f), sg(NH, 0.03f);
    if (cudaMemcpy(w.data(), weights, w.size() * sizeof(float), cudaMemcpyDeviceToHost) != cudaSuccess ||
        slime_ca_set_weights(cached, 0, w.data(), w.data() + wn, w.data() + 2 * wn, wo.data(), k.data(), mu.data(), sg.data()) ||
        slime_ca_set_state_device(cached, ca_state, SLIME_CA_F32, nullptr) || slime_ca_step(cached, 1, nullptr)) {
        fprintf(stderr, "launch_multi_head_ca: %s\n", slime_ca_last_error(cached));
        return;
    }
    void* vp = nullptr;
    size_t bytes = 0;
    slime_ca_buffer(cached, SLIME_CA_BUF_VPRIME_LAST, &vp, &bytes);
    if (cudaMemcpy(ca_output, vp, bytes, cudaMemcpyDeviceToDevice) != cudaSuccess || cudaDeviceSynchronize() != cudaSuccess)
        fprintf(stderr, "launch_multi_head_ca: %s\n", cudaGetErrorString(cudaGetLastError()));
}

}  // extern "C"

// ---------------------------------------------------------------------------------------------------------------
// Row-stripe ring, occupancy, elite record, bounded-wait self-test.

namespace {

// The reference's genome hash (gpu_sha256, slime/memory/archive.cu:41-60: despite the name a 64-bit
// shift-add-xor mix over the fp32 bit patterns, one value after the other), restated.
unsigned long long genome_hash(const float* genome, size_t n) {
    unsigned long long hsh = 0x9e3779b97f4a7c15ULL;
    for (size_t i = 0; i < n; ++i) {
        unsigned int bits;
        memcpy(&bits, genome + i, sizeof bits);
        hsh ^= (unsigned long long)(unsigned int)(bits + 0x9e3779b9u) + (hsh << 6) + (hsh >> 2);   // 32-bit sum, wrapping
        hsh += hsh << 3;
        hsh ^= hsh >> 11;
        hsh += hsh << 15;
        hsh *= 0xc4ceb9fe1a85ec53ULL;
        hsh ^= hsh >> 33;
    }
    return hsh;
}

// One thread waits, with the limit it is given, on an mbarrier nobody will ever arrive on, and reports that.
__global__ void k_wait_selftest(int* status, unsigned long long limit_ns, int code) {
    __shared__ uint64_t bar;
    if (threadIdx.x == 0) {
        ptx::mbar_init(&bar, 1);
        ptx::fence_barrier_init();
        ptx::mbar_wait(&bar, 0, status, code, limit_ns);
        ptx::mbar_inval(&bar);
    }
}

// n_steps ring steps; ev (optional) gets 4 events per step: before the exchange, after it, after the kernels and
// the local reduction, after the all-reduce and the new scale
int ring_steps(slime_ca* h, int n_steps, cudaStream_t st, std::vector<cudaEvent_t>* ev) {
    const int n = h->g.B * NC;
    for (int i = 0; i < n_steps; ++i) {
        int rc;
        if (ev) CK(h, cudaEventRecord((*ev)[(size_t)i * 4], st));
        if ((rc = ring_exchange(h, st))) return rc;
        if (ev) CK(h, cudaEventRecord((*ev)[(size_t)i * 4 + 1], st));
        void* emit = nullptr;
        if (h->cfg.keep_vprime && i >= n_steps - 2) { h->vp_last ^= 1; emit = h->vprime[h->vp_last]; ++h->vp_steps; h->fitness_valid = false; }
        if ((rc = step_kernels(h, emit, st))) return rc;
        if (ev) CK(h, cudaEventRecord((*ev)[(size_t)i * 4 + 2], st));
        if ((rc = ring_allreduce(h, h->sums, st))) return rc;
        k_scale_from_sums<<<(n + 255) / 256, 256, 0, st>>>(h->sums, h->mass, h->scale, n);
        LAUNCHED(h);
        if (ev) CK(h, cudaEventRecord((*ev)[(size_t)i * 4 + 3], st));
        ++h->steps_done;
    }
    return SLIME_CA_OK;
}

}  // namespace

extern "C" {

int slime_ca_ring_unique_id(void* id_out) {
    if (!id_out) return SLIME_CA_EINVAL;
    const nccl::Api& n = nccl::api();
    if (!n.ok) return SLIME_CA_ECOMM;
    nccl::unique_id id;
    if (n.GetUniqueId(&id) != nccl::SUCCESS) return SLIME_CA_ECOMM;
    memcpy(id_out, &id, sizeof id);
    return SLIME_CA_OK;
}

static int ring_check_handle(slime_ca* h, int rank, int world) {
    if (!h) return SLIME_CA_EINVAL;
    if (!h->cfg.stripe) return fail(h, SLIME_CA_ESTATE, "a ring needs a handle created in stripe mode");
    if (world < 1 || rank < 0 || rank >= world) return fail(h, SLIME_CA_EINVAL, "bad rank or world size");
    if (h->g.H < 3) return fail(h, SLIME_CA_EINVAL, "a stripe needs at least 3 own rows (the halo is 3 rows)");
    return SLIME_CA_OK;
}

int slime_ca_ring_init(slime_ca* h, const void* id, int rank, int world) {
    int rc = ring_check_handle(h, rank, world);
    if (rc) return rc;
    ring_release(h);
    CK(h, cudaSetDevice(h->cfg.device));
    if (world > 1) {
        if (!id) return fail(h, SLIME_CA_EINVAL, "null unique id");
        const nccl::Api& n = nccl::api();
        if (!n.ok) return fail(h, SLIME_CA_ECOMM, n.error);
        nccl::unique_id uid;
        memcpy(&uid, id, sizeof uid);
        nccl::comm_t comm = nullptr;
        NK(h, n.CommInitRank(&comm, world, uid, rank));
        h->comm = comm;
        h->own_comm = true;
    }
    h->ring_rank = rank;
    h->ring_world = world;
    return SLIME_CA_OK;
}

int slime_ca_ring_attach(slime_ca* h, void* nccl_comm, int rank, int world) {
    int rc = ring_check_handle(h, rank, world);
    if (rc) return rc;
    ring_release(h);
    if (world > 1) {
        if (!nccl_comm) return fail(h, SLIME_CA_EINVAL, "null communicator");
        const nccl::Api& n = nccl::api();
        if (!n.ok) return fail(h, SLIME_CA_ECOMM, n.error);
        int count = 0, me = -1;
        NK(h, n.CommCount((nccl::comm_t)nccl_comm, &count));
        NK(h, n.CommUserRank((nccl::comm_t)nccl_comm, &me));
        if (count != world || me != rank) return fail(h, SLIME_CA_EINVAL, "rank / world size do not match the communicator");
        h->comm = nccl_comm;
        h->own_comm = false;
    }
    h->ring_rank = rank;
    h->ring_world = world;
    return SLIME_CA_OK;
}

int slime_ca_ring_detach(slime_ca* h) {
    if (!h) return SLIME_CA_EINVAL;
    ring_release(h);
    return SLIME_CA_OK;
}

int slime_ca_ring_sync_mass(slime_ca* h, void* stream) {
    int rc = ring_ready(h);
    if (rc) return rc;
    CK(h, cudaSetDevice(h->cfg.device));
    return ring_allreduce(h, h->mass, (cudaStream_t)stream);
}

int slime_ca_step_ring(slime_ca* h, int n_steps, void* stream) {
    int rc = ring_ready(h);
    if (rc) return rc;
    if (n_steps < 0) return fail(h, SLIME_CA_EINVAL, "negative step count");
    CK(h, cudaSetDevice(h->cfg.device));
    cudaStream_t st = (cudaStream_t)stream;
    if ((rc = poll_status(h, st))) return rc;
    if ((rc = ring_steps(h, n_steps, st, nullptr))) return rc;
    return n_steps > 0 ? publish_status(h, st) : SLIME_CA_OK;
}

int slime_ca_step_ring_timed(slime_ca* h, int n_steps, void* stream, float* ms) {
    int rc = ring_ready(h);
    if (rc) return rc;
    if (n_steps <= 0 || n_steps > 4096 || !ms) return fail(h, SLIME_CA_EINVAL, "bad step count or null output");
    CK(h, cudaSetDevice(h->cfg.device));
    cudaStream_t st = (cudaStream_t)stream;
    struct Events {
        std::vector<cudaEvent_t> v;
        ~Events() { for (cudaEvent_t e : v) if (e) cudaEventDestroy(e); }
    } evs;
    evs.v.assign((size_t)n_steps * 4, nullptr);
    for (auto& e : evs.v) CK(h, cudaEventCreate(&e));
    if ((rc = ring_steps(h, n_steps, st, &evs.v))) return rc;
    CK(h, cudaStreamSynchronize(st));
    ms[0] = ms[1] = ms[2] = 0.f;
    for (int i = 0; i < n_steps; ++i)
        for (int k = 0; k < 3; ++k) {
            float t = 0.f;
            CK(h, cudaEventElapsedTime(&t, evs.v[(size_t)i * 4 + k], evs.v[(size_t)i * 4 + k + 1]));
            ms[k] += t;
        }
    return check_status_word(h);
}

int slime_ca_ring_wait(slime_ca* h, void* stream, int timeout_ms) {
    if (!h) return SLIME_CA_EINVAL;
    if (timeout_ms < 0) return fail(h, SLIME_CA_EINVAL, "negative timeout");
    CK(h, cudaSetDevice(h->cfg.device));
    cudaStream_t st = (cudaStream_t)stream;
    const auto deadline = std::chrono::steady_clock::now() + std::chrono::milliseconds(timeout_ms);
    for (;;) {
        const cudaError_t q = cudaStreamQuery(st);
        if (q == cudaSuccess) return check_status_word(h);
        if (q != cudaErrorNotReady) return fail(h, SLIME_CA_ECUDA, std::string("cudaStreamQuery: ") + cudaGetErrorString(q));
        if (h->comm) {
            int async = nccl::SUCCESS;
            const nccl::Api& n = nccl::api();
            if (n.CommGetAsyncError((nccl::comm_t)h->comm, &async) == nccl::SUCCESS && async != nccl::SUCCESS &&
                async != nccl::IN_PROGRESS) {
                n.CommAbort((nccl::comm_t)h->comm);      // frees the communicator and ends its kernels
                h->comm = nullptr; h->own_comm = false; h->ring_world = 0;
                return fail(h, SLIME_CA_ECOMM, "the ring's communicator reported " + nccl::describe(async) + "; it was aborted");
            }
        }
        if (std::chrono::steady_clock::now() >= deadline) {
            if (h->comm) {
                nccl::api().CommAbort((nccl::comm_t)h->comm);
                h->comm = nullptr; h->own_comm = false; h->ring_world = 0;
                return fail(h, SLIME_CA_ETIMEOUT, "the stream did not drain within " + std::to_string(timeout_ms) +
                                                      " ms; the ring's communicator was aborted (attach a new one to go on)");
            }
            return fail(h, SLIME_CA_ETIMEOUT, "the stream did not drain within " + std::to_string(timeout_ms) + " ms");
        }
        std::this_thread::sleep_for(std::chrono::microseconds(200));
    }
}

int slime_ca_selftest_bounded_wait(slime_ca* h, unsigned long long limit_ns, void* stream) {
    if (!h) return SLIME_CA_EINVAL;
    if (limit_ns == 0 || limit_ns > 100000000ull) return fail(h, SLIME_CA_EINVAL, "limit must lie in (0, 100 ms]");
    CK(h, cudaSetDevice(h->cfg.device));
    cudaStream_t st = (cudaStream_t)stream;
    k_wait_selftest<<<1, 32, 0, st>>>(h->dev_status, limit_ns, 901);
    LAUNCHED(h);
    return publish_status(h, st);
}

int slime_ca_occupancy(slime_ca* h, float* occupancy) {
    if (!h) return SLIME_CA_EINVAL;
    if (!occupancy) return fail(h, SLIME_CA_EINVAL, "null output pointer");
    CK(h, cudaSetDevice(h->cfg.device));
    int max_threads = 0;
    CK(h, cudaDeviceGetAttribute(&max_threads, cudaDevAttrMaxThreadsPerMultiProcessor, h->cfg.device));
    int b1 = 0, b2 = 0, t1, t2;
    if (is_bf16(h)) {
        t1 = k1b::THREADS; t2 = k2m::THREADS;
        if (h->bf.k1_aligned) CK(h, cudaOccupancyMaxActiveBlocksPerMultiprocessor(&b1, k1_bf16<true>, t1, k1b::SMEM));
        else CK(h, cudaOccupancyMaxActiveBlocksPerMultiprocessor(&b1, k1_bf16<false>, t1, k1b::SMEM));
        CK(h, cudaOccupancyMaxActiveBlocksPerMultiprocessor(&b2, k2_bf16, t2, k2m::SMEM));
    } else {
        t1 = t2 = 256;
        CK(h, cudaOccupancyMaxActiveBlocksPerMultiprocessor(&b1, k1_f32, t1, K1F32_SMEM));
        CK(h, cudaOccupancyMaxActiveBlocksPerMultiprocessor(&b2, k2_f32, t2, K2F32_SMEM));
    }
    const float o1 = (float)(b1 * t1) / (float)max_threads, o2 = (float)(b2 * t2) / (float)max_threads;
    *occupancy = o1 < o2 ? o1 : o2;
    return SLIME_CA_OK;
}

int slime_ca_elite_record(slime_ca* h, int set_index, int generation, slime_ca_elite* out, void* stream) {
    int rc = ready(h);
    if (rc) return rc;
    if (!out) return fail(h, SLIME_CA_EINVAL, "null output pointer");
    if (set_index < 0 || set_index >= h->cfg.n_weight_sets) return fail(h, SLIME_CA_EINVAL, "weight set index out of range");
    if (!h->cfg.keep_vprime || !h->fitness_valid)
        return fail(h, SLIME_CA_ESTATE, "the elite record follows slime_ca_fitness on the same state");
    CK(h, cudaSetDevice(h->cfg.device));
    cudaStream_t st = (cudaStream_t)stream;
    const int per = h->g.per_set;
    std::vector<float> fit((size_t)per * 4), genome(MW_STRIDE);
    int parent = set_index;
    CK(h, cudaMemcpyAsync(fit.data(), h->fit_dev + (size_t)set_index * per * 4, fit.size() * sizeof(float), cudaMemcpyDeviceToHost, st));
    CK(h, cudaMemcpyAsync(genome.data(), h->master + (size_t)set_index * MW_STRIDE, genome.size() * sizeof(float), cudaMemcpyDeviceToHost, st));
    CK(h, cudaMemcpyAsync(&parent, h->parent + set_index, sizeof(int), cudaMemcpyDeviceToHost, st));
    CK(h, cudaStreamSynchronize(st));
    double s[3] = {0, 0, 0};
    for (int i = 0; i < per; ++i) { s[0] += fit[i * 4 + 2]; s[1] += fit[i * 4 + 1]; s[2] += fit[i * 4 + 0]; }
    memset(out, 0, sizeof *out);
    out->fitness = (float)(s[0] / per);
    out->coherence = (float)(s[1] / per);
    out->effective_rank = (float)(s[2] / per);
    out->genome_hash = genome_hash(genome.data(), genome.size());
    const unsigned int par = h->evolved ? (unsigned int)parent : (unsigned int)set_index;
    out->parent_ids[0] = par;
    out->parent_ids[1] = par;          // refills copy one parent (no crossover): both slots name it
    out->generation = (unsigned short)(generation & 0xffff);
    return SLIME_CA_OK;
}

}  // extern "C"

// ---------------------------------------------------------------------------------------------------------------
// Per-channel sums without any allocation.
//
// Some callers of this library can not allocate device memory at the point where they need a state's channel
// masses: a host loop that has handed the whole device to its own pool (a framework's caching allocator, or the
// reference's habit of carving every buffer out of pools made once in create_organism, slime/runtime.cu:275-326),
// where a cudaMalloc simply fails, and latency-critical generation loops, where the implicit device-wide
// synchronisation of cudaMalloc / cudaFree is not acceptable.  For them the two-stage reduction below keeps its
// scratch (the per-chunk partial sums) in a fixed array that is part of the loaded library image.
//
// The array is a file-scope __device__ object: every GPU that loads the library holds its 2 MiB until the process
// exits.  In host code its name is only a handle for the runtime, not a device address, so the address is looked up
// once per device with cudaGetSymbolAddress (below) and that pointer is what the kernels receive.
constexpr int STATIC_MAX_CHUNKS = 8192;    // 256-cell chunks over all grids of one call: at most 2 097 152 cells
static __device__ __align__(256) float g_static_partials[(size_t)STATIC_MAX_CHUNKS * NC];

namespace {
constexpr int STATIC_MAX_DEVICES = 64;
std::atomic<float*> g_static_partials_addr[STATIC_MAX_DEVICES] = {};
thread_local std::string g_static_error;

int static_fail(int code, const std::string& msg) {
    g_static_error = msg;
    return code;
}
}  // namespace

extern "C" {

const char* slime_ca_static_error(void) { return g_static_error.c_str(); }

int slime_ca_channel_sums_static(const void* dev_state, int dtype, int batch, int cells_per_grid, double* dev_sums,
                                 void* stream) {
    if (!dev_state || !dev_sums) return static_fail(SLIME_CA_EINVAL, "null pointer");
    if (dtype != SLIME_CA_F32 && dtype != SLIME_CA_BF16) return static_fail(SLIME_CA_EINVAL, "dtype must be SLIME_CA_F32 or SLIME_CA_BF16");
    if (batch <= 0 || cells_per_grid <= 0) return static_fail(SLIME_CA_EINVAL, "batch and cells_per_grid must be positive");
    const long long chunks = ((long long)cells_per_grid + 255) / 256;
    if (chunks * batch > STATIC_MAX_CHUNKS)
        return static_fail(SLIME_CA_EINVAL, "too large for the built-in scratch: batch * ceil(cells_per_grid / 256) = " +
                                                std::to_string(chunks * batch) + " exceeds " + std::to_string(STATIC_MAX_CHUNKS) +
                                                " (use a handle and slime_ca_get_mass instead)");
    int dev = -1;
    cudaError_t e = cudaGetDevice(&dev);
    if (e != cudaSuccess) return static_fail(SLIME_CA_ECUDA, std::string("cudaGetDevice: ") + cudaGetErrorString(e));
    if (dev < 0 || dev >= STATIC_MAX_DEVICES) return static_fail(SLIME_CA_EINVAL, "device ordinal out of range");
    if (!g_static_partials_addr[dev].load(std::memory_order_acquire)) {
        // set-up, once per device, with that device current: resolve the device address of the scratch array
        float* p = nullptr;
        e = cudaGetSymbolAddress((void**)&p, g_static_partials);
        if (e != cudaSuccess || !p) return static_fail(SLIME_CA_ECUDA, std::string("cudaGetSymbolAddress: ") + cudaGetErrorString(e));
        g_static_partials_addr[dev].store(p, std::memory_order_release);   // two first callers store the same address
    }
    float* partial = g_static_partials_addr[dev].load(std::memory_order_acquire);
    cudaStream_t st = (cudaStream_t)stream;
    Geom g{};
    g.B = batch; g.H = cells_per_grid; g.W = 1; g.hx = 0; g.he = 0; g.wrap_y = 1; g.per_set = 1;
    const dim3 grid((unsigned)chunks, (unsigned)batch);
    if (dtype == SLIME_CA_BF16) k_channel_partials<__nv_bfloat16><<<grid, 256, 0, st>>>((const __nv_bfloat16*)dev_state, partial, g);
    else k_channel_partials<float><<<grid, 256, 0, st>>>((const float*)dev_state, partial, g);
    e = cudaGetLastError();
    if (e != cudaSuccess) return static_fail(SLIME_CA_ECUDA, std::string("kernel launch: ") + cudaGetErrorString(e));
    // one segment per grid: the fp64 second stage writes [batch][64] straight into the caller's buffer
    k_reduce_partials<<<dim3(1, (unsigned)batch), 256, 0, st>>>(partial, (int)chunks, dev_sums);
    e = cudaGetLastError();
    if (e != cudaSuccess) return static_fail(SLIME_CA_ECUDA, std::string("kernel launch: ") + cudaGetErrorString(e));
    g_static_error.clear();
    return SLIME_CA_OK;
}

}  // extern "C"

