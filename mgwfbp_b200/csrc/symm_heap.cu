// Symmetric heap: each rank owns one device allocation of identical layout and maps every
// peer's allocation into its own address space, so kernels can load from and store to any GPU of
// the NVSwitch box with ordinary global-memory instructions.
//
// Two implementations behind the same idea:
//
//  * VMM heap (default): physical memory from cuMemCreate, exported as a POSIX file descriptor,
//    imported and mapped by every peer with cuMemMap.  Because the memory is a VMM allocation it
//    can additionally be BOUND TO AN NVSWITCH MULTICAST OBJECT (cuMulticastCreate / AddDevice /
//    BindMem): one more virtual range then addresses "the same offset on every GPU", which is what
//    the multimem.ld_reduce / multimem.st instructions of the NVLS all-reduce operate on.  File
//    descriptors travel between the processes over a Unix socket owned by the Python side.
//  * IPC heap (fallback, and the one the failure tests use): cudaMalloc + cudaIpc handles, 64-byte
//    blobs over the host control plane, no multicast.
//
// The driver entry points are resolved through the runtime (cudaGetDriverEntryPoint), so the
// library does not link against libcuda and still loads on a machine without a driver.
#include <cuda.h>
#include <cstdio>
#include <cstring>
#include <unistd.h>
#include "api.h"

static thread_local char g_last_error[512] = "";

extern "C" void mgw_set_last_error(cudaError_t e, const char* what, const char* file, int line) {
    snprintf(g_last_error, sizeof(g_last_error), "%s failed at %s:%d: %s (%s)", what, file, line,
             cudaGetErrorString(e), cudaGetErrorName(e));
    (void)cudaGetLastError();   // clear the sticky-free error so later calls start clean
}

extern "C" void mgw_set_last_error_text(const char* text) {
    snprintf(g_last_error, sizeof(g_last_error), "%s", text);
}

extern "C" const char* mgw_last_error(void) { return g_last_error; }
extern "C" int mgw_version(void) { return 200; }

// ------------------------------------------------------------------------------------------------
// IPC heap
// ------------------------------------------------------------------------------------------------
extern "C" int mgw_heap_create(size_t bytes, void** base_out) {
    if (base_out == nullptr || bytes == 0) return MGW_ERR_ARG;
    void* p = nullptr;
    MGW_CUDA_CHECK(cudaMalloc(&p, bytes));
    MGW_CUDA_CHECK(cudaMemset(p, 0, bytes));
    MGW_CUDA_CHECK(cudaDeviceSynchronize());
    *base_out = p;
    return MGW_OK;
}

extern "C" int mgw_heap_export(void* base, void* handle64_out) {
    static_assert(sizeof(cudaIpcMemHandle_t) == 64, "IPC handle size");
    cudaIpcMemHandle_t h;
    MGW_CUDA_CHECK(cudaIpcGetMemHandle(&h, base));
    memcpy(handle64_out, &h, sizeof(h));
    return MGW_OK;
}

extern "C" int mgw_heap_open(const void* handle64, void** peer_base_out) {
    cudaIpcMemHandle_t h;
    memcpy(&h, handle64, sizeof(h));
    void* p = nullptr;
    MGW_CUDA_CHECK(cudaIpcOpenMemHandle(&p, h, cudaIpcMemLazyEnablePeerAccess));
    *peer_base_out = p;
    return MGW_OK;
}

extern "C" int mgw_heap_close(void* peer_base) {
    MGW_CUDA_CHECK(cudaIpcCloseMemHandle(peer_base));
    return MGW_OK;
}

extern "C" int mgw_heap_destroy(void* base) {
    MGW_CUDA_CHECK(cudaFree(base));
    return MGW_OK;
}

extern "C" int mgw_host_status_alloc(int n_ints, int** host_ptr_out) {
    int* p = nullptr;
    MGW_CUDA_CHECK(cudaHostAlloc((void**)&p, sizeof(int) * (size_t)n_ints, cudaHostAllocMapped | cudaHostAllocPortable));
    memset(p, 0, sizeof(int) * (size_t)n_ints);
    *host_ptr_out = p;
    return MGW_OK;
}

extern "C" int mgw_host_status_free(int* host_ptr) {
    MGW_CUDA_CHECK(cudaFreeHost(host_ptr));
    return MGW_OK;
}

// ------------------------------------------------------------------------------------------------
// VMM heap with optional NVSwitch multicast binding
// ------------------------------------------------------------------------------------------------
namespace {

struct DriverApi {
    bool ready = false;
    CUresult (*GetErrorString)(CUresult, const char**) = nullptr;
    CUresult (*DeviceGet)(CUdevice*, int) = nullptr;
    CUresult (*DeviceGetAttribute)(int*, CUdevice_attribute, CUdevice) = nullptr;
    CUresult (*MemGetAllocationGranularity)(size_t*, const CUmemAllocationProp*, CUmemAllocationGranularity_flags) = nullptr;
    CUresult (*MemCreate)(CUmemGenericAllocationHandle*, size_t, const CUmemAllocationProp*, unsigned long long) = nullptr;
    CUresult (*MemRelease)(CUmemGenericAllocationHandle) = nullptr;
    CUresult (*MemAddressReserve)(CUdeviceptr*, size_t, size_t, CUdeviceptr, unsigned long long) = nullptr;
    CUresult (*MemAddressFree)(CUdeviceptr, size_t) = nullptr;
    CUresult (*MemMap)(CUdeviceptr, size_t, size_t, CUmemGenericAllocationHandle, unsigned long long) = nullptr;
    CUresult (*MemUnmap)(CUdeviceptr, size_t) = nullptr;
    CUresult (*MemSetAccess)(CUdeviceptr, size_t, const CUmemAccessDesc*, size_t) = nullptr;
    CUresult (*MemExportToShareableHandle)(void*, CUmemGenericAllocationHandle, CUmemAllocationHandleType, unsigned long long) = nullptr;
    CUresult (*MemImportFromShareableHandle)(CUmemGenericAllocationHandle*, void*, CUmemAllocationHandleType) = nullptr;
    CUresult (*MulticastCreate)(CUmemGenericAllocationHandle*, const CUmulticastObjectProp*) = nullptr;
    CUresult (*MulticastAddDevice)(CUmemGenericAllocationHandle, CUdevice) = nullptr;
    CUresult (*MulticastBindMem)(CUmemGenericAllocationHandle, size_t, CUmemGenericAllocationHandle, size_t, size_t, unsigned long long) = nullptr;
    CUresult (*MulticastUnbind)(CUmemGenericAllocationHandle, CUdevice, size_t, size_t) = nullptr;
    CUresult (*MulticastGetGranularity)(size_t*, const CUmulticastObjectProp*, CUmulticastGranularity_flags) = nullptr;
};

DriverApi g_drv;

template <typename F>
bool resolve(const char* name, F& fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint(name, &p, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess || p == nullptr) {
        (void)cudaGetLastError();
        char buf[160];
        snprintf(buf, sizeof(buf), "driver entry point %s is not available", name);
        mgw_set_last_error_text(buf);
        return false;
    }
    fn = reinterpret_cast<F>(p);
    return true;
}

bool driver_ready() {
    if (g_drv.ready) return true;
    if (cudaFree(nullptr) != cudaSuccess) {             // make sure a context exists on the current device
        mgw_set_last_error(cudaGetLastError(), "cudaFree(0)", __FILE__, __LINE__);
        return false;
    }
    DriverApi d;
    bool ok = resolve("cuGetErrorString", d.GetErrorString) && resolve("cuDeviceGet", d.DeviceGet) &&
              resolve("cuDeviceGetAttribute", d.DeviceGetAttribute) &&
              resolve("cuMemGetAllocationGranularity", d.MemGetAllocationGranularity) && resolve("cuMemCreate", d.MemCreate) &&
              resolve("cuMemRelease", d.MemRelease) && resolve("cuMemAddressReserve", d.MemAddressReserve) &&
              resolve("cuMemAddressFree", d.MemAddressFree) && resolve("cuMemMap", d.MemMap) && resolve("cuMemUnmap", d.MemUnmap) &&
              resolve("cuMemSetAccess", d.MemSetAccess) && resolve("cuMemExportToShareableHandle", d.MemExportToShareableHandle) &&
              resolve("cuMemImportFromShareableHandle", d.MemImportFromShareableHandle) &&
              resolve("cuMulticastCreate", d.MulticastCreate) && resolve("cuMulticastAddDevice", d.MulticastAddDevice) &&
              resolve("cuMulticastBindMem", d.MulticastBindMem) && resolve("cuMulticastUnbind", d.MulticastUnbind) &&
              resolve("cuMulticastGetGranularity", d.MulticastGetGranularity);
    if (!ok) return false;
    d.ready = true;
    g_drv = d;
    return true;
}

#define MGW_CU_CHECK(expr)                                                                          \
    do {                                                                                            \
        CUresult _r = (expr);                                                                       \
        if (_r != CUDA_SUCCESS) {                                                                   \
            const char* _s = nullptr;                                                               \
            if (g_drv.GetErrorString) g_drv.GetErrorString(_r, &_s);                                \
            char _buf[400];                                                                         \
            snprintf(_buf, sizeof(_buf), "%s failed at %s:%d: %s (CUresult %d)", #expr, __FILE__, __LINE__, \
                     _s ? _s : "?", (int)_r);                                                       \
            mgw_set_last_error_text(_buf);                                                          \
            return MGW_ERR_CUDA;                                                                    \
        }                                                                                           \
    } while (0)

struct VmmHeap {
    int device = 0;
    CUdevice cu_device = 0;
    size_t bytes = 0;                        // rounded up to the granularity in use
    size_t granularity = 0;
    CUmemGenericAllocationHandle local = 0;
    CUdeviceptr base = 0;
    CUmemGenericAllocationHandle peer_handle[MGW_MAX_RANKS] = {};
    CUdeviceptr peer_va[MGW_MAX_RANKS] = {};
    CUmemGenericAllocationHandle mc = 0;
    bool mc_have = false, mc_added = false, mc_bound = false;
    CUdeviceptr mc_va = 0;
};

CUmemAllocationProp local_prop(int device) {
    CUmemAllocationProp prop;
    memset(&prop, 0, sizeof(prop));
    prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
    prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
    prop.location.id = device;
    prop.requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
    return prop;
}

int map_rw(CUdeviceptr* va_out, size_t bytes, size_t align, CUmemGenericAllocationHandle h, int device) {
    CUdeviceptr va = 0;
    MGW_CU_CHECK(g_drv.MemAddressReserve(&va, bytes, align, 0, 0));
    CUresult r = g_drv.MemMap(va, bytes, 0, h, 0);
    if (r != CUDA_SUCCESS) {
        g_drv.MemAddressFree(va, bytes);
        MGW_CU_CHECK(r);
    }
    CUmemAccessDesc acc;
    memset(&acc, 0, sizeof(acc));
    acc.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
    acc.location.id = device;
    acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
    r = g_drv.MemSetAccess(va, bytes, &acc, 1);
    if (r != CUDA_SUCCESS) {
        g_drv.MemUnmap(va, bytes);
        g_drv.MemAddressFree(va, bytes);
        MGW_CU_CHECK(r);
    }
    *va_out = va;
    return MGW_OK;
}

}  // namespace

// out2[0]: 1 when VMM allocations with POSIX file-descriptor handles work on the current device,
// out2[1]: 1 when the device can additionally join an NVSwitch multicast object.
extern "C" int mgw_vmm_supported(int* out2) {
    if (out2 == nullptr) return MGW_ERR_ARG;
    out2[0] = out2[1] = 0;
    if (!driver_ready()) return MGW_ERR_CUDA;
    int dev = 0;
    MGW_CUDA_CHECK(cudaGetDevice(&dev));
    CUdevice cd;
    MGW_CU_CHECK(g_drv.DeviceGet(&cd, dev));
    int vmm = 0, fd = 0, mc = 0;
    MGW_CU_CHECK(g_drv.DeviceGetAttribute(&vmm, CU_DEVICE_ATTRIBUTE_VIRTUAL_MEMORY_MANAGEMENT_SUPPORTED, cd));
    MGW_CU_CHECK(g_drv.DeviceGetAttribute(&fd, CU_DEVICE_ATTRIBUTE_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR_SUPPORTED, cd));
    MGW_CU_CHECK(g_drv.DeviceGetAttribute(&mc, CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED, cd));
    out2[0] = (vmm && fd) ? 1 : 0;
    out2[1] = (vmm && fd && mc) ? 1 : 0;
    return MGW_OK;
}

// Allocate and map this rank's part.  `bytes` is rounded up to the allocation granularity (to the
// multicast granularity of a `world`-device object when want_multicast is set, so that the whole
// allocation can be bound); the rounded size is returned and must be equal on every rank.
extern "C" int mgw_vmm_create(size_t bytes, int world, int want_multicast, void** heap_out, void** base_out, size_t* bytes_out) {
    if (heap_out == nullptr || base_out == nullptr || bytes_out == nullptr || bytes == 0 || world < 1 || world > MGW_MAX_RANKS)
        return MGW_ERR_ARG;
    if (!driver_ready()) return MGW_ERR_CUDA;
    VmmHeap* h = new VmmHeap();
    MGW_CUDA_CHECK(cudaGetDevice(&h->device));
    MGW_CU_CHECK(g_drv.DeviceGet(&h->cu_device, h->device));
    CUmemAllocationProp prop = local_prop(h->device);
    size_t gran = 0;
    MGW_CU_CHECK(g_drv.MemGetAllocationGranularity(&gran, &prop, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED));
    if (want_multicast && world > 1) {
        CUmulticastObjectProp mp;
        memset(&mp, 0, sizeof(mp));
        mp.numDevices = (unsigned)world;
        mp.size = bytes;
        mp.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
        size_t mg = 0;
        MGW_CU_CHECK(g_drv.MulticastGetGranularity(&mg, &mp, CU_MULTICAST_GRANULARITY_RECOMMENDED));
        if (mg > gran) gran = mg;
    }
    h->granularity = gran;
    h->bytes = (bytes + gran - 1) / gran * gran;
    CUresult r = g_drv.MemCreate(&h->local, h->bytes, &prop, 0);
    if (r != CUDA_SUCCESS) { delete h; MGW_CU_CHECK(r); }
    int rc = map_rw(&h->base, h->bytes, gran, h->local, h->device);
    if (rc != MGW_OK) { g_drv.MemRelease(h->local); delete h; return rc; }
    MGW_CUDA_CHECK(cudaMemset((void*)h->base, 0, h->bytes));
    MGW_CUDA_CHECK(cudaDeviceSynchronize());
    *heap_out = h;
    *base_out = (void*)h->base;
    *bytes_out = h->bytes;
    return MGW_OK;
}

// A file descriptor for this rank's allocation (the caller sends it to the peers and closes it).
extern "C" int mgw_vmm_export_fd(void* heap, int* fd_out) {
    VmmHeap* h = static_cast<VmmHeap*>(heap);
    if (h == nullptr || fd_out == nullptr) return MGW_ERR_ARG;
    int fd = -1;
    MGW_CU_CHECK(g_drv.MemExportToShareableHandle(&fd, h->local, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0));
    *fd_out = fd;
    return MGW_OK;
}

// Map the allocation of rank `peer` (its descriptor as received over the Unix socket; closed here).
extern "C" int mgw_vmm_import_peer(void* heap, int peer, int fd, void** peer_base_out) {
    VmmHeap* h = static_cast<VmmHeap*>(heap);
    if (h == nullptr || peer < 0 || peer >= MGW_MAX_RANKS || fd < 0 || peer_base_out == nullptr) return MGW_ERR_ARG;
    CUmemGenericAllocationHandle ph = 0;
    CUresult r = g_drv.MemImportFromShareableHandle(&ph, (void*)(uintptr_t)fd, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR);
    close(fd);
    MGW_CU_CHECK(r);
    CUdeviceptr va = 0;
    int rc = map_rw(&va, h->bytes, h->granularity, ph, h->device);
    if (rc != MGW_OK) { g_drv.MemRelease(ph); return rc; }
    h->peer_handle[peer] = ph;
    h->peer_va[peer] = va;
    *peer_base_out = (void*)va;
    return MGW_OK;
}

// Multicast object: created by one rank (fd_out = descriptor to hand to the others) ...
extern "C" int mgw_vmm_mc_create(void* heap, int world, int* fd_out) {
    VmmHeap* h = static_cast<VmmHeap*>(heap);
    if (h == nullptr || fd_out == nullptr || world < 2) return MGW_ERR_ARG;
    CUmulticastObjectProp mp;
    memset(&mp, 0, sizeof(mp));
    mp.numDevices = (unsigned)world;
    mp.size = h->bytes;
    mp.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
    MGW_CU_CHECK(g_drv.MulticastCreate(&h->mc, &mp));
    h->mc_have = true;
    int fd = -1;
    MGW_CU_CHECK(g_drv.MemExportToShareableHandle(&fd, h->mc, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0));
    *fd_out = fd;
    return MGW_OK;
}

// ... imported by the others (the descriptor is closed here) ...
extern "C" int mgw_vmm_mc_import(void* heap, int fd) {
    VmmHeap* h = static_cast<VmmHeap*>(heap);
    if (h == nullptr || fd < 0) return MGW_ERR_ARG;
    CUresult r = g_drv.MemImportFromShareableHandle(&h->mc, (void*)(uintptr_t)fd, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR);
    close(fd);
    MGW_CU_CHECK(r);
    h->mc_have = true;
    return MGW_OK;
}

// ... joined by every rank's device (all ranks must have done this before any of them binds) ...
extern "C" int mgw_vmm_mc_add_device(void* heap) {
    VmmHeap* h = static_cast<VmmHeap*>(heap);
    if (h == nullptr || !h->mc_have) return MGW_ERR_ARG;
    MGW_CU_CHECK(g_drv.MulticastAddDevice(h->mc, h->cu_device));
    h->mc_added = true;
    return MGW_OK;
}

// ... and finally bound to this rank's allocation and mapped.  mc_base_out + off then addresses offset
// `off` of every rank's allocation at once (multimem instructions only).
extern "C" int mgw_vmm_mc_bind(void* heap, void** mc_base_out) {
    VmmHeap* h = static_cast<VmmHeap*>(heap);
    if (h == nullptr || !h->mc_added || mc_base_out == nullptr) return MGW_ERR_ARG;
    MGW_CU_CHECK(g_drv.MulticastBindMem(h->mc, 0, h->local, 0, h->bytes, 0));
    h->mc_bound = true;
    int rc = map_rw(&h->mc_va, h->bytes, h->granularity, h->mc, h->device);
    if (rc != MGW_OK) return rc;
    *mc_base_out = (void*)h->mc_va;
    return MGW_OK;
}

// Undo everything this rank did, in reverse order.  Call it on every rank after a host barrier behind the
// last kernel that touched the heap.  `what`: 1 = only the multicast part, 0 = everything.
extern "C" int mgw_vmm_destroy(void* heap, int what) {
    VmmHeap* h = static_cast<VmmHeap*>(heap);
    if (h == nullptr) return MGW_ERR_ARG;
    if (!g_drv.ready) return MGW_ERR_CUDA;
    (void)cudaDeviceSynchronize();
    if (h->mc_va) { g_drv.MemUnmap(h->mc_va, h->bytes); g_drv.MemAddressFree(h->mc_va, h->bytes); h->mc_va = 0; }
    if (h->mc_bound) { g_drv.MulticastUnbind(h->mc, h->cu_device, 0, h->bytes); h->mc_bound = false; }
    if (h->mc_have) { g_drv.MemRelease(h->mc); h->mc_have = false; h->mc_added = false; }
    if (what == 1) return MGW_OK;
    for (int r = 0; r < MGW_MAX_RANKS; ++r) {
        if (h->peer_va[r]) {
            g_drv.MemUnmap(h->peer_va[r], h->bytes);
            g_drv.MemAddressFree(h->peer_va[r], h->bytes);
            g_drv.MemRelease(h->peer_handle[r]);
            h->peer_va[r] = 0;
        }
    }
    if (h->base) {
        g_drv.MemUnmap(h->base, h->bytes);
        g_drv.MemAddressFree(h->base, h->bytes);
        g_drv.MemRelease(h->local);
        h->base = 0;
    }
    delete h;
    return MGW_OK;
}
