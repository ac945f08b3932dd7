// Cache partitions that other processes can map: physical memory from the CUDA virtual memory
// management API, exported as a POSIX file descriptor and mapped by every peer with explicit
// read access.  One process per GPU replaces the reference's one thread per GPU
// (sampling_server/src/engine/server.cu:127-135), so the pointer table of the clique
// (cache/cache.cu:601-622) has to cross process boundaries.  Legacy CUDA IPC handles work too
// (legion_ipc_get_handle / legion_ipc_open_handle) but random 512-byte reads through such a mapping
// fell to ~75 GB/s on an 11 GB partition, against ~640 GB/s through a mapping made here.
//
// The driver entry points are looked up at run time, so the library does not link libcuda.
#include "common.cuh"

#include <cuda.h>
#include <stdlib.h>
#include <unistd.h>

namespace legion {

struct Driver {
    CUresult (*GetGranularity)(size_t *, const CUmemAllocationProp *, CUmemAllocationGranularity_flags);
    CUresult (*Create)(CUmemGenericAllocationHandle *, size_t, const CUmemAllocationProp *, unsigned long long);
    CUresult (*Export)(void *, CUmemGenericAllocationHandle, CUmemAllocationHandleType, unsigned long long);
    CUresult (*Import)(CUmemGenericAllocationHandle *, void *, CUmemAllocationHandleType);
    CUresult (*Reserve)(CUdeviceptr *, size_t, size_t, CUdeviceptr, unsigned long long);
    CUresult (*Map)(CUdeviceptr, size_t, size_t, CUmemGenericAllocationHandle, unsigned long long);
    CUresult (*SetAccess)(CUdeviceptr, size_t, const CUmemAccessDesc *, size_t);
    CUresult (*Unmap)(CUdeviceptr, size_t);
    CUresult (*Release)(CUmemGenericAllocationHandle);
    CUresult (*AddressFree)(CUdeviceptr, size_t);
    bool ok;
};

static bool load_one(const char *name, void **fn)
{
    cudaDriverEntryPointQueryResult q;
    return cudaGetDriverEntryPoint(name, fn, cudaEnableDefault, &q) == cudaSuccess && q == cudaDriverEntryPointSuccess &&
           *fn != nullptr;
}

static Driver *driver()
{
    static Driver d;
    static bool tried = false;
    if (!tried) {
        tried = true;
        d.ok = load_one("cuMemGetAllocationGranularity", (void **)&d.GetGranularity) &&
               load_one("cuMemCreate", (void **)&d.Create) &&
               load_one("cuMemExportToShareableHandle", (void **)&d.Export) &&
               load_one("cuMemImportFromShareableHandle", (void **)&d.Import) &&
               load_one("cuMemAddressReserve", (void **)&d.Reserve) && load_one("cuMemMap", (void **)&d.Map) &&
               load_one("cuMemSetAccess", (void **)&d.SetAccess) && load_one("cuMemUnmap", (void **)&d.Unmap) &&
               load_one("cuMemRelease", (void **)&d.Release) && load_one("cuMemAddressFree", (void **)&d.AddressFree);
    }
    return &d;
}

static CUmemAllocationProp prop_of(int dev)
{
    CUmemAllocationProp prop;
    memset(&prop, 0, sizeof(prop));
    prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
    prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
    prop.location.id = dev;
    prop.requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
    return prop;
}

#define LG_DRV(call, what)                                                              \
    do {                                                                                \
        CUresult r_ = (call);                                                           \
        if (r_ != CUDA_SUCCESS) {                                                       \
            set_error("%s:%d: %s failed with CUresult %d", __FILE__, __LINE__, what, (int)r_); \
            return LEGION_E_CUDA;                                                       \
        }                                                                               \
    } while (0)

// Allocates `bytes` (rounded up to the allocation granularity) on `dev`, mapped read-write for it.
int vmm_alloc(int dev, int64_t bytes, VmmBlock *out)
{
    Driver *d = driver();
    // LEGION_NO_VMM=1 stands for a platform without the virtual memory management API (tests of the
    // cudaMalloc + peer-access fallback)
    const char *off = getenv("LEGION_NO_VMM");
    if (!d->ok || (off != nullptr && off[0] == '1')) {
        set_error("CUDA virtual memory management entry points are not available");
        return LEGION_E_STATE;
    }
    LG_CUDA(cudaSetDevice(dev));
    LG_CUDA(cudaFree(0));  // make sure the primary context exists
    CUmemAllocationProp prop = prop_of(dev);
    size_t gran = 0;
    LG_DRV(d->GetGranularity(&gran, &prop, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED), "cuMemGetAllocationGranularity");
    size_t size = ((size_t)bytes + gran - 1) / gran * gran;
    CUmemGenericAllocationHandle h;
    LG_DRV(d->Create(&h, size, &prop, 0), "cuMemCreate");
    CUdeviceptr ptr = 0;
    if (d->Reserve(&ptr, size, gran, 0, 0) != CUDA_SUCCESS) {
        d->Release(h);
        set_error("cuMemAddressReserve failed");
        return LEGION_E_NOMEM;
    }
    CUmemAccessDesc acc;
    memset(&acc, 0, sizeof(acc));
    acc.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
    acc.location.id = dev;
    acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
    if (d->Map(ptr, size, 0, h, 0) != CUDA_SUCCESS || d->SetAccess(ptr, size, &acc, 1) != CUDA_SUCCESS) {
        d->AddressFree(ptr, size);
        d->Release(h);
        set_error("cuMemMap / cuMemSetAccess failed");
        return LEGION_E_CUDA;
    }
    out->ptr = (void *)ptr;
    out->size = (int64_t)size;
    out->handle = (unsigned long long)h;
    out->imported = 0;
    return LEGION_OK;
}

int vmm_export_fd(const VmmBlock *b, int *fd_out)
{
    Driver *d = driver();
    int fd = -1;
    LG_DRV(d->Export(&fd, (CUmemGenericAllocationHandle)b->handle, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0),
           "cuMemExportToShareableHandle");
    *fd_out = fd;
    return LEGION_OK;
}

// Maps another process's block (received as a file descriptor) with read access for `dev`.
int vmm_import_fd(int dev, int fd, int64_t size, VmmBlock *out)
{
    Driver *d = driver();
    if (!d->ok) {
        set_error("CUDA virtual memory management entry points are not available");
        return LEGION_E_STATE;
    }
    LG_CUDA(cudaSetDevice(dev));
    LG_CUDA(cudaFree(0));
    CUmemAllocationProp prop = prop_of(dev);
    size_t gran = 0;
    LG_DRV(d->GetGranularity(&gran, &prop, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED), "cuMemGetAllocationGranularity");
    CUmemGenericAllocationHandle h;
    LG_DRV(d->Import(&h, (void *)(uintptr_t)fd, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR), "cuMemImportFromShareableHandle");
    CUdeviceptr ptr = 0;
    if (d->Reserve(&ptr, (size_t)size, gran, 0, 0) != CUDA_SUCCESS) {
        d->Release(h);
        set_error("cuMemAddressReserve failed");
        return LEGION_E_NOMEM;
    }
    CUmemAccessDesc acc;
    memset(&acc, 0, sizeof(acc));
    acc.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
    acc.location.id = dev;
    acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READ;
    CUresult r1 = d->Map(ptr, (size_t)size, 0, h, 0);
    CUresult r2 = r1 == CUDA_SUCCESS ? d->SetAccess(ptr, (size_t)size, &acc, 1) : r1;
    if (r2 != CUDA_SUCCESS) {
        if (r1 == CUDA_SUCCESS) d->Unmap(ptr, (size_t)size);
        d->AddressFree(ptr, (size_t)size);
        d->Release(h);
        set_error("mapping a peer partition failed with CUresult %d (is peer access possible between the GPUs?)", (int)r2);
        return LEGION_E_CUDA;
    }
    out->ptr = (void *)ptr;
    out->size = size;
    out->handle = (unsigned long long)h;
    out->imported = 1;
    return LEGION_OK;
}

void vmm_free(VmmBlock *b)
{
    if (b->ptr == nullptr) return;
    Driver *d = driver();
    d->Unmap((CUdeviceptr)b->ptr, (size_t)b->size);
    d->AddressFree((CUdeviceptr)b->ptr, (size_t)b->size);
    d->Release((CUmemGenericAllocationHandle)b->handle);
    b->ptr = nullptr;
}

}  // namespace legion

using namespace legion;

// The clique's pointer table across processes (cache/cache.cu:601-622): export this GPU's partition
// as a file descriptor (send it over a unix socket with SCM_RIGHTS; the caller closes it) ...
extern "C" int legion_cache_export_partition(LegionCache *c, int32_t *fd_out, int64_t *bytes_out)
{
    LG_ARG(c != nullptr && c->kind == 0 && fd_out != nullptr && bytes_out != nullptr, "not a static cache");
    if (c->own_block.ptr == nullptr) {
        set_error("legion_cache_export_partition: the partition was not allocated as shareable memory");
        return LEGION_E_STATE;
    }
    int fd = -1;
    int rc = vmm_export_fd(&c->own_block, &fd);
    if (rc != LEGION_OK) return rc;
    *fd_out = fd;
    *bytes_out = c->own_block.size;
    return LEGION_OK;
}

// ... and map member k's partition from the descriptor received from its process.
extern "C" int legion_cache_import_peer(LegionCache *c, int32_t k, int32_t fd, int64_t bytes)
{
    LG_ARG(c != nullptr && c->kind == 0, "not a static cache");
    LG_ARG(k >= 0 && k < c->kg && k != c->ki, "k must name another member of the clique");
    LG_ARG(fd >= 0 && bytes > 0, "bad descriptor or size");
    if (c->peer_block[k].ptr != nullptr) vmm_free(&c->peer_block[k]);
    int rc = vmm_import_fd(c->dev_id, fd, bytes, &c->peer_block[k]);
    if (rc != LEGION_OK) return rc;
    c->part[k] = c->peer_block[k].ptr;
    return LEGION_OK;
}

// One process, one thread per GPU (the reference's layout, engine/server.cu:127-135): lets device
// `dev` read this cache's partition in place; the other thread then passes legion_cache_partition's
// pointer to legion_cache_set_peer.  Ordinary cudaMalloc partitions use legion_enable_peer_access.
extern "C" int legion_cache_allow_device(LegionCache *c, int32_t dev)
{
    LG_ARG(c != nullptr && c->kind == 0 && dev >= 0, "not a static cache");
    if (dev == c->dev_id) return LEGION_OK;
    if (c->own_block.ptr == nullptr) {
        // the partition is ordinary cudaMalloc memory (no virtual memory management on this platform):
        // device `dev` reads it through peer access, or the call fails; it never reports success without
        // either, because the gather would then dereference a pointer that `dev` cannot reach
        int cur = -1;
        LG_CUDA(cudaGetDevice(&cur));
        int rc = legion_enable_peer_access(dev, c->dev_id);
        if (cur >= 0) cudaSetDevice(cur);
        return rc;
    }
    Driver *d = driver();
    CUmemAccessDesc acc;
    memset(&acc, 0, sizeof(acc));
    acc.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
    acc.location.id = dev;
    acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READ;
    LG_DRV(d->SetAccess((CUdeviceptr)c->own_block.ptr, (size_t)c->own_block.size, &acc, 1), "cuMemSetAccess");
    return LEGION_OK;
}
