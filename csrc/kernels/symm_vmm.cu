// Symmetric memory from the virtual-memory-management API, with an NVLink multicast object on top.
//
// The cudaMalloc + CUDA-IPC heap (runtime.cu) gives every rank plain peer pointers. This file adds the second kind:
// every rank creates its region with cuMemCreate, exports it as a POSIX file descriptor, maps every peer's region
// into its own address space, and binds its region to ONE multicast object that rank 0 created for the group. The
// multicast object is mapped too; a `multimem.st` to that mapping is replicated by the NVSwitch into the region of
// every rank (one store on the sender's links instead of one per peer), and `multimem.ld_reduce` reads and combines
// all replicas inside the switch. The low-latency all-gather pushes through it (allgather.cu).
//
// File descriptors travel between the ranks on Unix sockets (SCM_RIGHTS), which the Python layer does
// (dlslime_b200/parallel/symm.py); this file only wraps the driver calls. The driver entry points are resolved at run
// time, so the library has no link-time dependency on libcuda and loads on machines without a GPU.
//
// Teardown order matters on NVSwitch systems: unmap the multicast mapping, unbind the device's memory from the
// multicast object and release it BEFORE the process exits or the region is freed; a rank that disappears while its
// memory is still bound can fault its peers' links.
#include "common/host_utils.h"
#include "slime_cuda.h"

using namespace slime;

namespace {

struct Driver {
    bool ok = false;
    CUresult (*MemCreate)(CUmemGenericAllocationHandle*, size_t, const CUmemAllocationProp*, unsigned long long) = nullptr;
    CUresult (*MemRelease)(CUmemGenericAllocationHandle)                                                          = nullptr;
    CUresult (*MemAddressReserve)(CUdeviceptr*, size_t, size_t, CUdeviceptr, unsigned long long)                  = nullptr;
    CUresult (*MemAddressFree)(CUdeviceptr, size_t)                                                               = nullptr;
    CUresult (*MemMap)(CUdeviceptr, size_t, size_t, CUmemGenericAllocationHandle, unsigned long long)             = nullptr;
    CUresult (*MemUnmap)(CUdeviceptr, size_t)                                                                     = nullptr;
    CUresult (*MemSetAccess)(CUdeviceptr, size_t, const CUmemAccessDesc*, size_t)                                 = nullptr;
    CUresult (*MemExport)(void*, CUmemGenericAllocationHandle, CUmemAllocationHandleType, unsigned long long)     = nullptr;
    CUresult (*MemImport)(CUmemGenericAllocationHandle*, void*, CUmemAllocationHandleType)                        = nullptr;
    CUresult (*MemGetGranularity)(size_t*, const CUmemAllocationProp*, CUmemAllocationGranularity_flags)          = nullptr;
    CUresult (*McCreate)(CUmemGenericAllocationHandle*, const CUmulticastObjectProp*)                             = nullptr;
    CUresult (*McAddDevice)(CUmemGenericAllocationHandle, CUdevice)                                               = nullptr;
    CUresult (*McBindMem)(CUmemGenericAllocationHandle, size_t, CUmemGenericAllocationHandle, size_t, size_t, unsigned long long) = nullptr;
    CUresult (*McUnbind)(CUmemGenericAllocationHandle, CUdevice, size_t, size_t)                                  = nullptr;
    CUresult (*McGetGranularity)(size_t*, const CUmulticastObjectProp*, CUmulticastGranularity_flags)             = nullptr;
    CUresult (*DeviceGetAttribute)(int*, CUdevice_attribute, CUdevice)                                            = nullptr;
};

template<typename F>
bool resolve(F& fn, const char* name)
{
    void*                           p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint(name, &p, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess || p == nullptr) {
        cudaGetLastError();
        return false;
    }
    fn = reinterpret_cast<F>(p);
    return true;
}

Driver& driver()
{
    static Driver d = [] {
        Driver x;
        x.ok = resolve(x.MemCreate, "cuMemCreate") && resolve(x.MemRelease, "cuMemRelease")
               && resolve(x.MemAddressReserve, "cuMemAddressReserve") && resolve(x.MemAddressFree, "cuMemAddressFree")
               && resolve(x.MemMap, "cuMemMap") && resolve(x.MemUnmap, "cuMemUnmap") && resolve(x.MemSetAccess, "cuMemSetAccess")
               && resolve(x.MemExport, "cuMemExportToShareableHandle") && resolve(x.MemImport, "cuMemImportFromShareableHandle")
               && resolve(x.MemGetGranularity, "cuMemGetAllocationGranularity") && resolve(x.McCreate, "cuMulticastCreate")
               && resolve(x.McAddDevice, "cuMulticastAddDevice") && resolve(x.McBindMem, "cuMulticastBindMem")
               && resolve(x.McUnbind, "cuMulticastUnbind") && resolve(x.McGetGranularity, "cuMulticastGetGranularity")
               && resolve(x.DeviceGetAttribute, "cuDeviceGetAttribute");
        return x;
    }();
    return d;
}

#define SLIME_CU_OK(expr)                                                                                              \
    do {                                                                                                               \
        CUresult _r = (expr);                                                                                          \
        if (_r != CUDA_SUCCESS) return ::slime::fail("%s failed with CUresult %d (%s:%d)", #expr, static_cast<int>(_r), __FILE__, __LINE__); \
    } while (0)

int current_device(int* dev)
{
    SLIME_CUDA_OK(cudaGetDevice(dev));
    SLIME_CUDA_OK(cudaFree(nullptr));  // makes sure the primary context exists and is current
    return 0;
}

CUmemAllocationProp alloc_prop(int dev)
{
    CUmemAllocationProp prop{};
    prop.type                 = CU_MEM_ALLOCATION_TYPE_PINNED;
    prop.location.type        = CU_MEM_LOCATION_TYPE_DEVICE;
    prop.location.id          = dev;
    prop.requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
    return prop;
}

int map_rw(Driver& d, CUmemGenericAllocationHandle h, unsigned long long bytes, unsigned long long align, int dev, CUdeviceptr* va_out)
{
    CUdeviceptr va = 0;
    SLIME_CU_OK(d.MemAddressReserve(&va, bytes, align, 0, 0));
    CUresult r = d.MemMap(va, bytes, 0, h, 0);
    if (r != CUDA_SUCCESS) {
        d.MemAddressFree(va, bytes);
        return fail("cuMemMap failed with CUresult %d", static_cast<int>(r));
    }
    CUmemAccessDesc acc{};
    acc.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
    acc.location.id   = dev;
    acc.flags         = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
    r                 = d.MemSetAccess(va, bytes, &acc, 1);
    if (r != CUDA_SUCCESS) {
        d.MemUnmap(va, bytes);
        d.MemAddressFree(va, bytes);
        return fail("cuMemSetAccess failed with CUresult %d", static_cast<int>(r));
    }
    *va_out = va;
    return 0;
}

}  // namespace

extern "C" {

// vmm: the device can export VMM allocations as file descriptors; multicast: it can join NVLink multicast objects.
int slime_vmm_support(int* vmm, int* multicast)
{
    *vmm = *multicast = 0;
    Driver& d = driver();
    if (!d.ok) return 0;
    int dev = 0;
    if (current_device(&dev)) return -1;
    int v = 0, m = 0;
    if (d.DeviceGetAttribute(&v, CU_DEVICE_ATTRIBUTE_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR_SUPPORTED, dev) == CUDA_SUCCESS) *vmm = v;
    if (d.DeviceGetAttribute(&m, CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED, dev) == CUDA_SUCCESS) *multicast = m;
    return 0;
}

// Smallest size >= bytes that both the allocation and a multicast object of `world` devices accept.
int slime_vmm_round_size(unsigned long long bytes, int world, int with_multicast, unsigned long long* rounded, unsigned long long* gran_out)
{
    Driver& d = driver();
    if (!d.ok) return fail("vmm: driver entry points not available");
    int dev = 0;
    if (current_device(&dev)) return -1;
    CUmemAllocationProp prop = alloc_prop(dev);
    size_t              gran = 0;
    SLIME_CU_OK(d.MemGetGranularity(&gran, &prop, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED));
    if (with_multicast) {
        CUmulticastObjectProp mp{};
        mp.numDevices  = static_cast<unsigned int>(world);
        mp.size        = bytes;
        mp.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
        size_t mg      = 0;
        SLIME_CU_OK(d.McGetGranularity(&mg, &mp, CU_MULTICAST_GRANULARITY_RECOMMENDED));
        if (mg > gran) gran = mg;
    }
    *gran_out = gran;
    *rounded  = (bytes + gran - 1) / gran * gran;
    return 0;
}

// This rank's region: created, mapped read/write, zeroed, exported. handle_out is the driver's allocation handle.
int slime_vmm_create(unsigned long long bytes, unsigned long long gran, unsigned long long* handle_out, void** va_out, int* fd_out)
{
    Driver& d = driver();
    if (!d.ok) return fail("vmm: driver entry points not available");
    int dev = 0;
    if (current_device(&dev)) return -1;
    CUmemAllocationProp          prop = alloc_prop(dev);
    CUmemGenericAllocationHandle h    = 0;
    SLIME_CU_OK(d.MemCreate(&h, bytes, &prop, 0));
    CUdeviceptr va = 0;
    if (map_rw(d, h, bytes, gran, dev, &va)) {
        d.MemRelease(h);
        return -1;
    }
    int      fd = -1;
    CUresult r  = d.MemExport(&fd, h, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0);
    if (r != CUDA_SUCCESS) {
        d.MemUnmap(va, bytes);
        d.MemAddressFree(va, bytes);
        d.MemRelease(h);
        return fail("cuMemExportToShareableHandle failed with CUresult %d", static_cast<int>(r));
    }
    SLIME_CUDA_OK(cudaMemset(reinterpret_cast<void*>(va), 0, bytes));
    SLIME_CUDA_OK(cudaDeviceSynchronize());
    *handle_out = h;
    *va_out     = reinterpret_cast<void*>(va);
    *fd_out     = fd;
    return 0;
}

// A peer's region from the file descriptor it exported (the descriptor stays the caller's to close).
int slime_vmm_import(int fd, unsigned long long bytes, unsigned long long gran, unsigned long long* handle_out, void** va_out)
{
    Driver& d = driver();
    if (!d.ok) return fail("vmm: driver entry points not available");
    int dev = 0;
    if (current_device(&dev)) return -1;
    CUmemGenericAllocationHandle h = 0;
    SLIME_CU_OK(d.MemImport(&h, reinterpret_cast<void*>(static_cast<uintptr_t>(fd)), CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR));
    CUdeviceptr va = 0;
    if (map_rw(d, h, bytes, gran, dev, &va)) {
        d.MemRelease(h);
        return -1;
    }
    *handle_out = h;
    *va_out     = reinterpret_cast<void*>(va);
    return 0;
}

int slime_vmm_unmap_release(unsigned long long handle, void* va, unsigned long long bytes)
{
    Driver& d = driver();
    if (!d.ok) return fail("vmm: driver entry points not available");
    if (va) {
        SLIME_CU_OK(d.MemUnmap(reinterpret_cast<CUdeviceptr>(va), bytes));
        SLIME_CU_OK(d.MemAddressFree(reinterpret_cast<CUdeviceptr>(va), bytes));
    }
    if (handle) SLIME_CU_OK(d.MemRelease(handle));
    return 0;
}

// Rank 0: the multicast object of the group, exported for the others.
int slime_vmm_mc_create(int world, unsigned long long bytes, unsigned long long* mc_out, int* fd_out)
{
    Driver& d = driver();
    if (!d.ok) return fail("vmm: driver entry points not available");
    int dev = 0;
    if (current_device(&dev)) return -1;
    CUmulticastObjectProp mp{};
    mp.numDevices  = static_cast<unsigned int>(world);
    mp.size        = bytes;
    mp.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
    CUmemGenericAllocationHandle mc = 0;
    SLIME_CU_OK(d.McCreate(&mc, &mp));
    int      fd = -1;
    CUresult r  = d.MemExport(&fd, mc, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0);
    if (r != CUDA_SUCCESS) {
        d.MemRelease(mc);
        return fail("export of the multicast object failed with CUresult %d", static_cast<int>(r));
    }
    *mc_out = mc;
    *fd_out = fd;
    return 0;
}

int slime_vmm_mc_import(int fd, unsigned long long* mc_out)
{
    Driver& d = driver();
    if (!d.ok) return fail("vmm: driver entry points not available");
    int dev = 0;
    if (current_device(&dev)) return -1;
    CUmemGenericAllocationHandle mc = 0;
    SLIME_CU_OK(d.MemImport(&mc, reinterpret_cast<void*>(static_cast<uintptr_t>(fd)), CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR));
    *mc_out = mc;
    return 0;
}

// Every rank, before anyone binds: this device joins the multicast object.
int slime_vmm_mc_add_device(unsigned long long mc)
{
    Driver& d = driver();
    if (!d.ok) return fail("vmm: driver entry points not available");
    int dev = 0;
    if (current_device(&dev)) return -1;
    SLIME_CU_OK(d.McAddDevice(mc, dev));
    return 0;
}

// After every rank has joined: bind this rank's region to the object and map the object.
int slime_vmm_mc_bind_map(unsigned long long mc, unsigned long long local_handle, unsigned long long bytes, unsigned long long gran,
                          void** mc_va_out)
{
    Driver& d = driver();
    if (!d.ok) return fail("vmm: driver entry points not available");
    int dev = 0;
    if (current_device(&dev)) return -1;
    SLIME_CU_OK(d.McBindMem(mc, 0, local_handle, 0, bytes, 0));
    CUdeviceptr va = 0;
    if (map_rw(d, mc, bytes, gran, dev, &va)) {
        d.McUnbind(mc, dev, 0, bytes);
        return -1;
    }
    *mc_va_out = reinterpret_cast<void*>(va);
    return 0;
}

// Teardown of this rank's share: unmap the object, unbind the region, drop the object handle.
int slime_vmm_mc_teardown(unsigned long long mc, void* mc_va, unsigned long long bytes, int bound)
{
    Driver& d = driver();
    if (!d.ok) return fail("vmm: driver entry points not available");
    int dev = 0;
    if (current_device(&dev)) return -1;
    if (mc_va) {
        SLIME_CU_OK(d.MemUnmap(reinterpret_cast<CUdeviceptr>(mc_va), bytes));
        SLIME_CU_OK(d.MemAddressFree(reinterpret_cast<CUdeviceptr>(mc_va), bytes));
    }
    if (bound) SLIME_CU_OK(d.McUnbind(mc, dev, 0, bytes));
    if (mc) SLIME_CU_OK(d.MemRelease(mc));
    return 0;
}

}  // extern "C"
