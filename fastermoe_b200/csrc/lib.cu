// Library-wide state: last-error text, device properties, version.
#include "common.cuh"
#include <cstring>
#include <mutex>

namespace fmoe {

static thread_local char g_err[512] = "";

void set_error(const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_err, sizeof(g_err), fmt, ap);
    va_end(ap);
}

int sm_count() {
    static int cached[64];
    static std::mutex mtx;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    std::lock_guard<std::mutex> lk(mtx);
    if (cached[dev] == 0) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0) n = 148;
        cached[dev] = n;
    }
    return cached[dev];
}

}  // namespace fmoe

extern "C" const char* fmoe_last_error_string(void) { return fmoe::g_err; }
extern "C" int fmoe_version(void) { return 100; }
extern "C" int fmoe_built_for_sm(void) { return 100; }

// Size in bytes of the structs that cross the C ABI, so that a binding written in another language can check
// its own declarations against the library it loaded (0: unknown name).
extern "C" size_t fmoe_abi_sizeof(const char* struct_name) {
    if (!struct_name) return 0;
    if (!strcmp(struct_name, "fmoe_move_t")) return sizeof(fmoe_move_t);
    if (!strcmp(struct_name, "fmoe_peer_seg_t")) return sizeof(fmoe_peer_seg_t);
    if (!strcmp(struct_name, "fmoe_arrival_t")) return sizeof(fmoe_arrival_t);
    if (!strcmp(struct_name, "fmoe_mlp_params_t")) return sizeof(fmoe_mlp_params_t);
    if (!strcmp(struct_name, "fmoe_fused_geometry_t")) return sizeof(fmoe_fused_geometry_t);
    return 0;
}
