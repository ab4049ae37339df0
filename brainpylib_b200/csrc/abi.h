// Opaque descriptor layouts and the status channel shared by every custom-call target.
//
// The structs are byte-identical (x86-64, natural alignment) to the reference's
// lib/kernel_helper_descriptor.cuh:49-144, lib/gpu_event_sum.cuh:10-41,
// lib/gpu_atomic_sum.cuh:10-13 and lib/gpu_atomic_prod.cuh:10-13, so a descriptor packed
// by either library is read correctly by the other.
#ifndef BPL_CSRC_ABI_H_
#define BPL_CSRC_ABI_H_

#include <cstddef>
#include <cstdint>
#include <cuda_runtime_api.h>

#include "../../include/brainpylib_b200.h"

namespace bpl {

struct TwoUintOneBoolDescriptor {  // 12 bytes (3 bytes of tail padding)
    unsigned int uint_x;
    unsigned int uint_y;
    bool bool_x;
};
struct DoubleSizeDescriptor {  // 8 bytes; also every legacy {conn_size|pre_size, post_size} descriptor
    unsigned int size_x;
    unsigned int size_y;
};
struct JITConnProbHomoDescriptor {  // 24 bytes (4 bytes of padding before prob)
    unsigned int n_row;
    unsigned int n_col;
    unsigned int seed;
    double prob;  // log(1 - conn_prob) for the v2 kernels
};
struct JITConnProbWeightedDescriptor {  // 40 bytes; the uniform and the normal descriptor share it
    unsigned int n_row;
    unsigned int n_col;
    unsigned int seed;
    double prob;
    double w1;  // uniform: w_min    normal: w_mu
    double w2;  // uniform: w_range  normal: w_sigma
};
struct MatMatJITProbDescriptor1 {  // 40 bytes
    unsigned int m;
    unsigned int k;
    unsigned int n;
    unsigned int seed;
    double log_p;
    double w1;
    double w2;
};

static_assert(sizeof(TwoUintOneBoolDescriptor) == 12, "layout");
static_assert(sizeof(DoubleSizeDescriptor) == 8, "layout");
static_assert(sizeof(JITConnProbHomoDescriptor) == 24 && offsetof(JITConnProbHomoDescriptor, prob) == 16, "layout");
static_assert(sizeof(JITConnProbWeightedDescriptor) == 40 && offsetof(JITConnProbWeightedDescriptor, w2) == 32, "layout");
static_assert(sizeof(MatMatJITProbDescriptor1) == 40 && offsetof(MatMatJITProbDescriptor1, log_p) == 16, "layout");

// Status of the last target call on this host thread (defined in gpu_ops.cc).
void set_status(int code, const char *message);
// bytes of the connection lists of the *_v1_ws matmat targets (jitconn_kernels.cu); elem = sizeof(T)
size_t matmat_list_workspace_bytes(const char *opaque, size_t opaque_len, size_t elem);

// The reference's UnpackDescriptor throws std::runtime_error("Invalid opaque object size")
// (lib/kernel_helpers.h:34-40); here the mismatch is recorded and the call returns.
template<typename D>
inline const D *unpack(const char *opaque, size_t opaque_len) {
    if (opaque == nullptr || opaque_len != sizeof(D)) {
        set_status(BPL_ERR_OPAQUE_SIZE, "Invalid opaque object size");
        return nullptr;
    }
    return reinterpret_cast<const D *>(opaque);
}

// After a launch: the reference's ThrowIfError(cudaGetLastError()) (lib/kernel_helpers_gpu.cuh:15-19).
inline bool launch_ok() {
    const cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) {
        set_status(BPL_ERR_CUDA, cudaGetErrorString(e));
        return false;
    }
    return true;
}

// Optional CUDA events recorded directly around the scatter kernel of a transposed event product (set with
// bpl_profile_scatter_events, per host thread, null = off).
cudaEvent_t profile_before();
cudaEvent_t profile_after();

// Number of SMs of the current device (cached per device; 148 on B200).
int sm_count();

inline bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15u) == 0; }

}  // namespace bpl

#endif  // BPL_CSRC_ABI_H_
