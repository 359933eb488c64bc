// A transform entry point for callers that must not allocate device memory.
//
// Some hosts of this library may not call cudaMalloc at the moment they need a transform: code running while a
// CUDA graph is being captured, real-time inference loops whose memory was carved up front, plug-ins that were
// handed a fixed device budget.  For them the scratch the transform needs (the operand between the longitude FFT
// and the Legendre contraction plus the degree slabs) lives in a device array that is part of the library image.
// The price: the array has a fixed size, every GPU that loads the library carries it until the process ends, and
// all calls share it.

#include <mutex>

#include "common.cuh"

struct shtb200_plan : public shtb200::Plan {};

namespace {

// 32 MiB: enough for e.g. a 91 x 180 grid with several hundred fields, or 721 x 1440 (lmax 720) with 3 fields.
constexpr size_t kStaticScratchBytes = SHTB200_STATIC_SCRATCH_BYTES;
static __device__ __align__(256) unsigned char g_static_scratch[kStaticScratchBytes];

constexpr int kMaxDevices = 64;
std::mutex g_setup_mutex;
void *g_scratch_addr[kMaxDevices] = {};

// The array's name is a host-side handle, not a device pointer; the address the kernels can use has to be asked
// for, once per device, with that device current.
int scratch_address(int device, void **out) {
    if (device < 0 || device >= kMaxDevices) return shtb200::fail(SHTB200_EINVAL, "device index out of range for the built-in scratch");
    std::lock_guard<std::mutex> lock(g_setup_mutex);
    if (!g_scratch_addr[device]) {
        void *p = nullptr;
        cudaError_t e = cudaGetSymbolAddress(&p, g_static_scratch);
        if (e != cudaSuccess || !p) return shtb200::fail(SHTB200_ECUDA, std::string("cudaGetSymbolAddress(static scratch): ") + cudaGetErrorString(e));
        g_scratch_addr[device] = p;
    }
    *out = g_scratch_addr[device];
    return SHTB200_OK;
}

}  // namespace

extern "C" {

size_t shtb200_static_scratch_bytes(void) { return kStaticScratchBytes; }

int shtb200_execute_static_scratch(shtb200_plan *plan, const void *in_dev, void *out_dev, int nfields, void *stream) {
    if (!plan) return shtb200::fail(SHTB200_EINVAL, "plan is null");
    if (nfields < 0) return shtb200::fail(SHTB200_EINVAL, "nfields must be >= 0");
    if (plan->profiling) return shtb200::fail(SHTB200_EINVAL, "per-kernel profiling creates CUDA events; switch it off before using the allocation-free call");
    const size_t need = shtb200_workspace_bytes(plan, nfields);
    if (need > kStaticScratchBytes)
        return shtb200::fail(SHTB200_EWORKSPACE, "this call needs " + std::to_string(need) + " bytes of scratch but the built-in array holds " +
                                                     std::to_string(kStaticScratchBytes) + "; use shtb200_execute with a caller-provided workspace");
    int prev = -1;
    if (cudaGetDevice(&prev) != cudaSuccess || cudaSetDevice(plan->device) != cudaSuccess) return shtb200::fail(SHTB200_ECUDA, "cudaSetDevice failed");
    void *scratch = nullptr;
    int rc = scratch_address(plan->device, &scratch);
    if (rc == SHTB200_OK) rc = shtb200_execute(plan, in_dev, out_dev, nfields, scratch, kStaticScratchBytes, stream);
    cudaSetDevice(prev);
    return rc;
}

}  // extern "C"
