// NCCL as the row-stripe ring's transport, bound at run time.
//
// The library has no link-time dependency on NCCL: the handful of entry points the ring needs are looked up in the
// NCCL the process already carries (a framework's bundled copy, or the caller's own) and only then in the system's
// libnccl.so.2, so a communicator made by the caller's NCCL is always driven by that same NCCL.  The declarations
// below restate the stable part of NCCL's public C interface (nccl.h): opaque communicator, 128-byte unique id,
// result / datatype / reduction codes.
#pragma once
#include <cuda_runtime.h>
#include <dlfcn.h>

#include <mutex>
#include <string>

namespace slime {
namespace nccl {

typedef struct ncclComm* comm_t;
struct unique_id { char internal[128]; };
constexpr int SUCCESS = 0, IN_PROGRESS = 7;
constexpr int DT_UINT8 = 1, DT_FLOAT64 = 8;     // ncclUint8, ncclFloat64
constexpr int OP_SUM = 0;                       // ncclSum

struct Api {
    int (*GetUniqueId)(unique_id*) = nullptr;
    int (*CommInitRank)(comm_t*, int, unique_id, int) = nullptr;
    int (*CommDestroy)(comm_t) = nullptr;
    int (*CommAbort)(comm_t) = nullptr;
    int (*CommGetAsyncError)(comm_t, int*) = nullptr;
    int (*CommCount)(comm_t, int*) = nullptr;
    int (*CommUserRank)(comm_t, int*) = nullptr;
    int (*GroupStart)() = nullptr;
    int (*GroupEnd)() = nullptr;
    int (*Send)(const void*, size_t, int, int, comm_t, cudaStream_t) = nullptr;
    int (*Recv)(void*, size_t, int, int, comm_t, cudaStream_t) = nullptr;
    int (*AllReduce)(const void*, void*, size_t, int, int, comm_t, cudaStream_t) = nullptr;
    const char* (*GetErrorString)(int) = nullptr;
    bool ok = false;
    std::string error;
};

inline const Api& api() {
    static Api a;
    static std::once_flag once;
    std::call_once(once, [] {
        void* lib = nullptr;
        auto sym = [&](const char* name) -> void* {
            void* p = dlsym(RTLD_DEFAULT, name);
            if (!p) {
                if (!lib) lib = dlopen("libnccl.so.2", RTLD_NOW | RTLD_GLOBAL);   // an already loaded copy is returned as is
                if (lib) p = dlsym(lib, name);
            }
            if (!p && a.error.empty()) a.error = std::string("NCCL entry point not found: ") + name;
            return p;
        };
#define SLIME_NCCL_BIND(field, name) a.field = reinterpret_cast<decltype(a.field)>(sym(name))
        SLIME_NCCL_BIND(GetUniqueId, "ncclGetUniqueId");
        SLIME_NCCL_BIND(CommInitRank, "ncclCommInitRank");
        SLIME_NCCL_BIND(CommDestroy, "ncclCommDestroy");
        SLIME_NCCL_BIND(CommAbort, "ncclCommAbort");
        SLIME_NCCL_BIND(CommGetAsyncError, "ncclCommGetAsyncError");
        SLIME_NCCL_BIND(CommCount, "ncclCommCount");
        SLIME_NCCL_BIND(CommUserRank, "ncclCommUserRank");
        SLIME_NCCL_BIND(GroupStart, "ncclGroupStart");
        SLIME_NCCL_BIND(GroupEnd, "ncclGroupEnd");
        SLIME_NCCL_BIND(Send, "ncclSend");
        SLIME_NCCL_BIND(Recv, "ncclRecv");
        SLIME_NCCL_BIND(AllReduce, "ncclAllReduce");
        SLIME_NCCL_BIND(GetErrorString, "ncclGetErrorString");
#undef SLIME_NCCL_BIND
        a.ok = a.error.empty();
    });
    return a;
}

inline std::string describe(int rc) {
    const Api& a = api();
    return a.GetErrorString ? std::string(a.GetErrorString(rc)) : ("NCCL result " + std::to_string(rc));
}

}  // namespace nccl
}  // namespace slime
