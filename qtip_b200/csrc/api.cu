// Status plumbing shared by the entry points.
#include "common.cuh"

namespace qtip {

static thread_local int g_last_cuda_error = 0;

void set_last_cuda_error(cudaError_t e) { g_last_cuda_error = (int)e; }

int sm_count() {
    static int cached[64] = {};
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess || dev < 0 || dev >= 64) return 148;
    if (cached[dev] == 0) {
        int v = 0;
        if (cudaDeviceGetAttribute(&v, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || v <= 0) v = 148;
        cached[dev] = v;
    }
    return cached[dev];
}

}  // namespace qtip

extern "C" const char *qtip_status_string(int status) {
    switch (status) {
        case QTIP_OK: return "ok";
        case QTIP_ERR_BAD_ARG: return "bad argument (null pointer, unsupported K / code / dtype, batch out of range)";
        case QTIP_ERR_BAD_SHAPE: return "unsupported shape";
        case QTIP_ERR_WORKSPACE: return "workspace missing or too small";
        case QTIP_ERR_CUDA: return "CUDA error (see qtip_last_cuda_error)";
        case QTIP_ERR_ALIGNMENT: return "pointer not aligned as required";
        case QTIP_ERR_TOO_LARGE: return "problem needs more scratch than the built-in array of qtip_decompress_matvec_static (4 MiB)";
        default: return "unknown status";
    }
}

extern "C" int qtip_last_cuda_error(void) { return qtip::g_last_cuda_error; }

extern "C" int qtip_version(void) { return 1; }
