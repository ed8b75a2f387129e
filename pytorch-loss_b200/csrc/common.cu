// Host-side plumbing of libb200loss: per-thread error string, launch checks,
// device queries and the tensor-map encoder (looked up in the driver at run time
// so the library links against the CUDA runtime only).
#include "common.cuh"

#include <string.h>
#include <atomic>

namespace b200 {

static thread_local char g_error[512] = "";
static std::atomic<uint64_t> g_launches{0};

void set_error(const char *fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof(g_error), fmt, ap);
    va_end(ap);
}

int launch_status(const char *what) {
    const cudaError_t e = cudaGetLastError();
    g_launches.fetch_add(1, std::memory_order_relaxed);
    if (e == cudaSuccess) return B200_OK;
    set_error("%s: %s", what, cudaGetErrorString(e));
    return B200_ERR_LAUNCH;
}

int sm_count() {
    static thread_local int cached_dev = -1, cached_sms = 0;
    int dev = 0;
    if (cudaGetDevice(&dev) != cudaSuccess) return 148;
    if (dev != cached_dev) {
        int n = 0;
        if (cudaDeviceGetAttribute(&n, cudaDevAttrMultiProcessorCount, dev) != cudaSuccess || n <= 0)
            n = 148;
        cached_dev = dev;
        cached_sms = n;
    }
    return cached_sms;
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *,
                                  const cuuint64_t *, const cuuint64_t *, const cuuint32_t *,
                                  const cuuint32_t *, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static EncodeTiledFn encode_fn() {
    static EncodeTiledFn fn = nullptr;
    static bool tried = false;
    if (!tried) {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) ==
                cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = reinterpret_cast<EncodeTiledFn>(p);
        tried = true;
    }
    return fn;
}

bool encode_tensor_map(CUtensorMap *map, int dtype, const void *base, int rank,
                       const uint64_t *dims, const uint64_t *strides_bytes, const uint32_t *box) {
    // The encoder is a driver call and needs a context bound to this thread; a thread that
    // has made no runtime call yet (e.g. a fresh autograd worker) has none.
    static thread_local bool context_bound = false;
    if (!context_bound) {
        cudaFree(nullptr);
        context_bound = true;
    }
    EncodeTiledFn fn = encode_fn();
    if (!fn) {
        set_error("cuTensorMapEncodeTiled is not available from this driver");
        return false;
    }
    cuuint64_t gdim[5];
    cuuint64_t gstr[5];
    cuuint32_t bdim[5];
    cuuint32_t estr[5];
    for (int i = 0; i < rank; ++i) {
        gdim[i] = dims[i];
        bdim[i] = box[i];
        estr[i] = 1;
        if (i > 0) gstr[i - 1] = strides_bytes[i];
    }
    CUtensorMapDataType dt;
    switch (dtype) {
        case B200_F32: dt = CU_TENSOR_MAP_DATA_TYPE_FLOAT32; break;
        case B200_F16: dt = CU_TENSOR_MAP_DATA_TYPE_FLOAT16; break;
        case B200_BF16: dt = CU_TENSOR_MAP_DATA_TYPE_BFLOAT16; break;
        default: dt = CU_TENSOR_MAP_DATA_TYPE_UINT32; break;   // raw 32-bit words
    }
    const CUresult r = fn(map, dt, static_cast<cuuint32_t>(rank), const_cast<void *>(base), gdim,
                          gstr, bdim, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                          CU_TENSOR_MAP_SWIZZLE_NONE, CU_TENSOR_MAP_L2_PROMOTION_L2_256B,
                          CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (r != CUDA_SUCCESS) {
        set_error("cuTensorMapEncodeTiled failed with CUresult %d", static_cast<int>(r));
        return false;
    }
    return true;
}

}  // namespace b200

namespace {
__global__ void set_exchange_kernel(void *workspace, const void *ctx) {
    *reinterpret_cast<const void **>(reinterpret_cast<char *>(workspace) + b200::kExchangeCtxOffset) = ctx;
}
}  // namespace

extern "C" {

int b200_abi_version(void) { return 3; }

uint64_t b200_kernel_launch_count(void) { return b200::g_launches.load(std::memory_order_relaxed); }

const char *b200_last_error(void) { return b200::g_error; }

size_t b200_reduce_workspace_bytes(void) { return b200::kReduceWorkspaceBytes; }

int b200_read_status(void *workspace, void *stream) {
    if (!workspace) {
        b200::set_error("b200_read_status: workspace is NULL");
        return B200_ERR_ARG;
    }
    cudaStream_t s = static_cast<cudaStream_t>(stream);
    unsigned status = 0;
    unsigned *word = reinterpret_cast<unsigned *>(workspace) + 1;
    if (cudaMemcpyAsync(&status, word, sizeof(status), cudaMemcpyDeviceToHost, s) != cudaSuccess ||
        cudaStreamSynchronize(s) != cudaSuccess) {
        return b200::launch_status("b200_read_status");
    }
    if (status == 0) return B200_OK;
    cudaMemsetAsync(word, 0, sizeof(unsigned), s);
    cudaStreamSynchronize(s);
    b200::set_error("device status word = 0x%x: a kernel gave up a bounded wait", status);
    return B200_ERR_STATUS;
}

size_t b200_exchange_ctx_bytes(void) { return sizeof(b200::ExchangeCtx); }
size_t b200_exchange_slot_bytes(int world) {
    return world > 0 ? size_t(b200::kExchangeSets) * size_t(world) * sizeof(b200::ExchangeSlot) : 0;
}

int b200_enable_peer_access(int peer_device) {
    int current = -1, can = 0;
    if (cudaGetDevice(&current) != cudaSuccess) return b200::launch_status("cudaGetDevice");
    if (peer_device == current) return B200_OK;
    if (cudaDeviceCanAccessPeer(&can, current, peer_device) != cudaSuccess || !can) {
        cudaGetLastError();
        b200::set_error("b200_enable_peer_access: device %d cannot access device %d", current, peer_device);
        return B200_ERR_UNSUPPORTED;
    }
    const cudaError_t e = cudaDeviceEnablePeerAccess(peer_device, 0);
    if (e != cudaSuccess && e != cudaErrorPeerAccessAlreadyEnabled) {
        cudaGetLastError();
        b200::set_error("b200_enable_peer_access: %s", cudaGetErrorString(e));
        return B200_ERR_UNSUPPORTED;
    }
    cudaGetLastError();     // "already enabled" is not an error to keep
    return B200_OK;
}

// CUDA IPC of the exchange slots.  The importer opens the handle with ITS OWN device current
// (cudaIpcMemLazyEnablePeerAccess): that maps the exporter's allocation into the importing
// device's address space, which is what kernels of that device need in order to store to it.
int b200_ipc_export(const void *dev_ptr, void *handle64, uint64_t *offset) {
    if (!dev_ptr || !handle64 || !offset) {
        b200::set_error("b200_ipc_export: null argument");
        return B200_ERR_ARG;
    }
    typedef CUresult (*RangeFn)(CUdeviceptr *, size_t *, CUdeviceptr);
    void *fp = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint("cuMemGetAddressRange", &fp, cudaEnableDefault, &q) != cudaSuccess ||
        q != cudaDriverEntryPointSuccess || !fp) {
        cudaGetLastError();
        b200::set_error("b200_ipc_export: cuMemGetAddressRange is not available");
        return B200_ERR_UNSUPPORTED;
    }
    cudaFree(nullptr);      // the driver call needs a context bound to this thread
    CUdeviceptr base = 0;
    size_t size = 0;
    if (reinterpret_cast<RangeFn>(fp)(&base, &size, reinterpret_cast<CUdeviceptr>(dev_ptr)) != CUDA_SUCCESS) {
        b200::set_error("b200_ipc_export: not a device allocation");
        return B200_ERR_ARG;
    }
    cudaIpcMemHandle_t h;
    static_assert(sizeof(h) == 64, "the handle travels as 64 bytes");
    const cudaError_t e = cudaIpcGetMemHandle(&h, reinterpret_cast<void *>(base));
    if (e != cudaSuccess) {
        cudaGetLastError();
        b200::set_error("b200_ipc_export: %s", cudaGetErrorString(e));
        return B200_ERR_UNSUPPORTED;
    }
    memcpy(handle64, &h, 64);
    *offset = uint64_t(reinterpret_cast<CUdeviceptr>(dev_ptr) - base);
    return B200_OK;
}

int b200_ipc_open(const void *handle64, uint64_t offset, void **mapped) {
    if (!handle64 || !mapped) {
        b200::set_error("b200_ipc_open: null argument");
        return B200_ERR_ARG;
    }
    cudaIpcMemHandle_t h;
    memcpy(&h, handle64, 64);
    void *base = nullptr;
    const cudaError_t e = cudaIpcOpenMemHandle(&base, h, cudaIpcMemLazyEnablePeerAccess);
    if (e != cudaSuccess) {
        cudaGetLastError();
        b200::set_error("b200_ipc_open: %s", cudaGetErrorString(e));
        return B200_ERR_UNSUPPORTED;
    }
    *mapped = static_cast<char *>(base) + offset;
    return B200_OK;
}

int b200_ipc_close(void *mapped, uint64_t offset) {
    if (!mapped) return B200_OK;
    const cudaError_t e = cudaIpcCloseMemHandle(static_cast<char *>(mapped) - offset);
    if (e != cudaSuccess) {
        cudaGetLastError();
        b200::set_error("b200_ipc_close: %s", cudaGetErrorString(e));
        return B200_ERR_ARG;
    }
    return B200_OK;
}

int b200_reduce_attach_exchange(void *workspace, const void *exchange_ctx, void *stream) {
    if (!workspace) {
        b200::set_error("b200_reduce_attach_exchange: workspace is NULL");
        return B200_ERR_ARG;
    }
    set_exchange_kernel<<<1, 1, 0, static_cast<cudaStream_t>(stream)>>>(workspace, exchange_ctx);
    return b200::launch_status("exchange attach launch");
}

}  // extern "C"
