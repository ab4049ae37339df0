// Registry, descriptor builders and status channel of the C ABI.
//
// Takes the place of the reference's pybind11 module lib/gpu_ops.cc (Registrations() :24-177,
// build_*_descriptor :181-198) and of lib/kernel_helper_descriptor.cu:13-102, but as plain
// `extern "C"` functions: the Python module `brainpylib_b200.gpu_ops` wraps the function
// pointers listed here in "xla._CUSTOM_CALL_TARGET" capsules itself.
#include <cstdio>
#include <cstring>

#include "abi.h"

namespace bpl {

namespace {
thread_local int g_status = BPL_OK;
thread_local char g_message[256] = {0};
}  // namespace

namespace {
thread_local cudaEvent_t g_profile_before = nullptr, g_profile_after = nullptr;
}  // namespace
cudaEvent_t profile_before() { return g_profile_before; }
cudaEvent_t profile_after() { return g_profile_after; }

void set_status(int code, const char *message) {
    g_status = code;
    std::snprintf(g_message, sizeof(g_message), "%s", message ? message : "");
}

int sm_count() {
    constexpr int MAX_DEVICES = 64;
    static int cached[MAX_DEVICES] = {0};   // 0 = unknown; a racing first call writes the same value
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 148;
    if (dev >= 0 && dev < MAX_DEVICES && cached[dev] > 0) return cached[dev];
    int n = 0;
    if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
    if (dev >= 0 && dev < MAX_DEVICES) cached[dev] = n;
    return n;
}

namespace {

struct Registration {
    const char *name;
    bpl_custom_call_t target;
};

#define BPL_REGISTRATION_ROW(name) {#name, &name},
const Registration kRegistrations[] = {BPL_FOR_EACH_TARGET(BPL_REGISTRATION_ROW)};
#undef BPL_REGISTRATION_ROW
constexpr int kRegistrationCount = static_cast<int>(sizeof(kRegistrations) / sizeof(kRegistrations[0]));

template<typename D>
size_t pack(const D &d, void *out, size_t cap) {
    if (out == nullptr || cap < sizeof(D)) return 0;
    std::memset(out, 0, sizeof(D));   // padding bytes are zero (the reference leaves them undefined)
    std::memcpy(out, &d, sizeof(D));
    return sizeof(D);
}

}  // namespace
}  // namespace bpl

using namespace bpl;

extern "C" {

size_t bpl_event_csr_workspace_bytes(uint32_t n_row, int transpose);   // csr_kernels.cu
size_t bpl_nonzero_workspace_bytes(uint32_t batch_size);               // event_info_kernels.cu

void bpl_profile_scatter_events(void *before, void *after) {
    g_profile_before = static_cast<cudaEvent_t>(before);
    g_profile_after = static_cast<cudaEvent_t>(after);
}

int bpl_last_status(char *message, size_t capacity) {
    if (message != nullptr && capacity > 0) std::snprintf(message, capacity, "%s", g_message);
    return g_status;
}

void bpl_clear_status(void) {
    g_status = BPL_OK;
    g_message[0] = 0;
}

int bpl_registration_count(void) { return kRegistrationCount; }
const char *bpl_registration_name(int i) {
    return (i >= 0 && i < kRegistrationCount) ? kRegistrations[i].name : nullptr;
}
bpl_custom_call_t bpl_registration_target(int i) {
    return (i >= 0 && i < kRegistrationCount) ? kRegistrations[i].target : nullptr;
}
bpl_custom_call_t bpl_find_target(const char *name) {
    if (name == nullptr) return nullptr;
    for (int i = 0; i < kRegistrationCount; ++i)
        if (std::strcmp(kRegistrations[i].name, name) == 0) return kRegistrations[i].target;
    return nullptr;
}

size_t bpl_workspace_bytes(const char *target_name, const char *opaque, size_t opaque_len) {
    if (target_name == nullptr) return 0;
    if (std::strncmp(target_name, "event_csr_matvec_", 17) == 0) {
        if (opaque == nullptr || opaque_len != sizeof(TwoUintOneBoolDescriptor)) return 0;
        const TwoUintOneBoolDescriptor *d = reinterpret_cast<const TwoUintOneBoolDescriptor *>(opaque);
        return bpl_event_csr_workspace_bytes(d->uint_x, d->bool_x ? 1 : 0);
    }
    if (std::strncmp(target_name, "event_cbcsr_matvec_", 19) == 0) {
        if (opaque == nullptr || opaque_len != 24) return 0;
        return bpl_event_csr_workspace_bytes(*reinterpret_cast<const uint32_t *>(opaque), 1);
    }
    if (std::strncmp(target_name, "gpu_matmat_prob_prob_", 21) == 0) {
        const size_t len = std::strlen(target_name);
        if (len < 6 || std::strcmp(target_name + len - 6, "_v1_ws") != 0) return 0;
        return bpl::matmat_list_workspace_bytes(opaque, opaque_len, std::strstr(target_name, "_double_") ? 8 : 4);
    }
    if (std::strncmp(target_name, "nonzero_", 8) == 0) {
        if (opaque == nullptr || opaque_len != sizeof(DoubleSizeDescriptor)) return 0;
        return bpl_nonzero_workspace_bytes(reinterpret_cast<const DoubleSizeDescriptor *>(opaque)->size_y);
    }
    return 0;
}

size_t bpl_build_twouint_onebool_descriptor(uint32_t uint_x, uint32_t uint_y, int bool_x, void *out, size_t cap) {
    TwoUintOneBoolDescriptor d;
    std::memset(&d, 0, sizeof(d));
    d.uint_x = uint_x; d.uint_y = uint_y; d.bool_x = bool_x != 0;
    return pack(d, out, cap);
}
size_t bpl_build_double_size_descriptor(uint32_t size_x, uint32_t size_y, void *out, size_t cap) {
    return pack(DoubleSizeDescriptor{size_x, size_y}, out, cap);
}
// The real-valued arguments are `float`, the fields `double`, exactly as in the reference
// (lib/kernel_helper_descriptor.cu:34-38): the kernels see float32-rounded values widened to double.
size_t bpl_build_jitconn_prob_homo_descriptor(uint32_t n_row, uint32_t n_col, uint32_t seed, float prob,
                                              void *out, size_t cap) {
    JITConnProbHomoDescriptor d;
    std::memset(&d, 0, sizeof(d));
    d.n_row = n_row; d.n_col = n_col; d.seed = seed; d.prob = prob;
    return pack(d, out, cap);
}
static size_t build_weighted(uint32_t n_row, uint32_t n_col, uint32_t seed, float prob, float w1, float w2,
                             void *out, size_t cap) {
    JITConnProbWeightedDescriptor d;
    std::memset(&d, 0, sizeof(d));
    d.n_row = n_row; d.n_col = n_col; d.seed = seed; d.prob = prob; d.w1 = w1; d.w2 = w2;
    return pack(d, out, cap);
}
size_t bpl_build_jitconn_prob_uniform_descriptor(uint32_t n_row, uint32_t n_col, uint32_t seed, float prob,
                                                 float w_min, float w_range, void *out, size_t cap) {
    return build_weighted(n_row, n_col, seed, prob, w_min, w_range, out, cap);
}
size_t bpl_build_jitconn_prob_normal_descriptor(uint32_t n_row, uint32_t n_col, uint32_t seed, float prob,
                                                float w_mu, float w_sigma, void *out, size_t cap) {
    return build_weighted(n_row, n_col, seed, prob, w_mu, w_sigma, out, cap);
}
size_t bpl_build_matmat_jit_prob_descriptor1(uint32_t m, uint32_t k, uint32_t n, uint32_t seed, float log_p,
                                             float w1, float w2, void *out, size_t cap) {
    MatMatJITProbDescriptor1 d;
    std::memset(&d, 0, sizeof(d));
    d.m = m; d.k = k; d.n = n; d.seed = seed; d.log_p = log_p; d.w1 = w1; d.w2 = w2;
    return pack(d, out, cap);
}
size_t bpl_build_csr_event_sum_descriptor(uint32_t pre_size, uint32_t post_size, void *out, size_t cap) {
    return pack(DoubleSizeDescriptor{pre_size, post_size}, out, cap);
}
size_t bpl_build_coo_event_sum_descriptor(uint32_t conn_size, uint32_t post_size, void *out, size_t cap) {
    return pack(DoubleSizeDescriptor{conn_size, post_size}, out, cap);
}
size_t bpl_build_coo_atomic_sum_descriptor(uint32_t conn_size, uint32_t post_size, void *out, size_t cap) {
    return pack(DoubleSizeDescriptor{conn_size, post_size}, out, cap);
}
size_t bpl_build_coo_atomic_prod_descriptor(uint32_t conn_size, uint32_t post_size, void *out, size_t cap) {
    return pack(DoubleSizeDescriptor{conn_size, post_size}, out, cap);
}
size_t bpl_build_nonzero_descriptor(uint32_t event_size, uint32_t batch_size, void *out, size_t cap) {
    return pack(DoubleSizeDescriptor{event_size, batch_size}, out, cap);
}

}  // extern "C"
