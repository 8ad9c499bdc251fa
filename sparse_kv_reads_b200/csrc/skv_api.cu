// Entry points shared by every kernel file: version, error text, cached device properties.
#include "skv_common.cuh"

namespace skv {

thread_local cudaError_t g_last_cuda_error = cudaSuccess;

struct DevProps {
    bool known = false;
    int sms = 0, smem_optin = 0;
};
static DevProps g_props[64];

static const DevProps &props() {
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) {
        static DevProps fallback;
        fallback.sms = 148;                // B200; only used to size grids when no device answers
        fallback.smem_optin = 227 * 1024;
        return fallback;
    }
    DevProps &p = g_props[dev];
    if (!p.known) {
        cudaDeviceGetAttribute(&p.sms, cudaDevAttrMultiProcessorCount, dev);
        cudaDeviceGetAttribute(&p.smem_optin, cudaDevAttrMaxSharedMemoryPerBlockOptin, dev);
        if (p.sms <= 0) p.sms = 148;
        if (p.smem_optin <= 0) p.smem_optin = 227 * 1024;
        p.known = true;
    }
    return p;
}

int device_sm_count() { return props().sms; }
static bool g_pdl = false;
bool pdl_enabled() {
    static const bool allowed = [] { const char *e = getenv("SKV_PDL"); return !(e && e[0] == '0'); }();
    return allowed && g_pdl;
}
int device_max_smem_optin() { return props().smem_optin; }

}  // namespace skv

extern "C" int skv_version(void) { return SKV_VERSION; }

extern "C" const char *skv_error_string(int code) {
    switch (code) {
        case SKV_OK: return "ok";
        case SKV_E_NULL: return "a required pointer is null";
        case SKV_E_DIM: return "unsupported head dimension, group size or slot count";
        case SKV_E_DTYPE: return "unknown element type";
        case SKV_E_ALIGN: return "pointer or stride is not 16-byte aligned";
        case SKV_E_RANGE: return "size or option out of range";
        case SKV_E_WORKSPACE: return "workspace too small";
        case SKV_E_CUDA: return "CUDA runtime error";
        case SKV_E_TOO_LARGE: return "request exceeds the fixed capacity of this entry point";
        default: return "unknown error code";
    }
}

extern "C" const char *skv_last_cuda_error(void) { return cudaGetErrorString(skv::g_last_cuda_error); }

extern "C" void skv_set_overlap(int on) { skv::g_pdl = on != 0; }
