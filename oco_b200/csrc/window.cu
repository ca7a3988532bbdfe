// Expert-parallel windows: one contiguous device address range of `world` slots, slot g backed by
// GPU g's memory (CUDA virtual memory management, handles passed between the ranks' processes as
// POSIX file descriptors). Rows that every rank keeps at the same offset of its own slot then have
// one global row number, slot * rows_per_slot + row, valid on every rank, so the expert stage gathers
// token rows from its peers and stores route outputs to them with the kernels it runs on one GPU:
// plain loads and stores over NVLink, no copy engine and no collective on the rows' way.
// The reference is single-device and has no counterpart.
#include <cuda.h>
#include <cuda_runtime.h>
#include <unistd.h>

#include <cstdarg>
#include <cstdio>
#include <vector>

#include "../../include/oco_moe.h"

namespace {

thread_local char g_error[256] = "";

int fail(int code, const char* fmt, ...) {
    va_list ap;
    va_start(ap, fmt);
    vsnprintf(g_error, sizeof g_error, fmt, ap);
    va_end(ap);
    return code;
}

template <typename Fn>
Fn driver_fn(const char* name) {
    void* fn = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint(name, &fn, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess) return nullptr;
    return (Fn)fn;
}

struct Driver {
    CUresult (*create)(CUmemGenericAllocationHandle*, size_t, const CUmemAllocationProp*, unsigned long long) = nullptr;
    CUresult (*release)(CUmemGenericAllocationHandle) = nullptr;
    CUresult (*granularity)(size_t*, const CUmemAllocationProp*, CUmemAllocationGranularity_flags) = nullptr;
    CUresult (*reserve)(CUdeviceptr*, size_t, size_t, CUdeviceptr, unsigned long long) = nullptr;
    CUresult (*address_free)(CUdeviceptr, size_t) = nullptr;
    CUresult (*map)(CUdeviceptr, size_t, size_t, CUmemGenericAllocationHandle, unsigned long long) = nullptr;
    CUresult (*unmap)(CUdeviceptr, size_t) = nullptr;
    CUresult (*set_access)(CUdeviceptr, size_t, const CUmemAccessDesc*, size_t) = nullptr;
    CUresult (*export_handle)(void*, CUmemGenericAllocationHandle, CUmemAllocationHandleType, unsigned long long) = nullptr;
    CUresult (*import_handle)(CUmemGenericAllocationHandle*, void*, CUmemAllocationHandleType) = nullptr;
    bool ok = false;
    Driver() {
        create = driver_fn<decltype(create)>("cuMemCreate");
        release = driver_fn<decltype(release)>("cuMemRelease");
        granularity = driver_fn<decltype(granularity)>("cuMemGetAllocationGranularity");
        reserve = driver_fn<decltype(reserve)>("cuMemAddressReserve");
        address_free = driver_fn<decltype(address_free)>("cuMemAddressFree");
        map = driver_fn<decltype(map)>("cuMemMap");
        unmap = driver_fn<decltype(unmap)>("cuMemUnmap");
        set_access = driver_fn<decltype(set_access)>("cuMemSetAccess");
        export_handle = driver_fn<decltype(export_handle)>("cuMemExportToShareableHandle");
        import_handle = driver_fn<decltype(import_handle)>("cuMemImportFromShareableHandle");
        ok = create && release && granularity && reserve && address_free && map && unmap && set_access && export_handle && import_handle;
    }
};

const Driver& driver() {
    static const Driver d;
    return d;
}

CUmemAllocationProp local_prop(int device) {
    CUmemAllocationProp prop{};
    prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
    prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
    prop.location.id = device;
    prop.requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
    return prop;
}

}  // namespace

struct oco_ep_window {
    int rank = 0, world = 0, device = 0;
    size_t stride = 0, backed = 0;
    CUdeviceptr base = 0;
    std::vector<CUmemGenericAllocationHandle> handles;
    std::vector<char> mapped;
    int fd = -1;
};

extern "C" {

const char* oco_ep_window_error(void) { return g_error; }

int oco_ep_window_granularity(size_t* bytes) {
    if (!bytes) return OCO_INVALID_ARGUMENT;
    const Driver& drv = driver();
    if (!drv.ok) return fail(OCO_CUDA_ERROR, "the driver's virtual memory calls are unavailable");
    int device = 0;
    if (cudaGetDevice(&device) != cudaSuccess) return fail(OCO_CUDA_ERROR, "no current device");
    CUmemAllocationProp prop = local_prop(device);
    CUresult r = drv.granularity(bytes, &prop, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED);
    if (r != CUDA_SUCCESS) return fail(OCO_CUDA_ERROR, "cuMemGetAllocationGranularity failed (%d)", (int)r);
    return OCO_OK;
}

int oco_ep_window_create(int rank, int world, size_t slot_stride, size_t backed_bytes, oco_ep_window** out) {
    if (!out || world < 1 || rank < 0 || rank >= world || backed_bytes == 0 || backed_bytes > slot_stride)
        return fail(OCO_INVALID_ARGUMENT, "bad rank, world or sizes");
    const Driver& drv = driver();
    if (!drv.ok) return fail(OCO_CUDA_ERROR, "the driver's virtual memory calls are unavailable");
    size_t gran = 0;
    if (int rc = oco_ep_window_granularity(&gran)) return rc;
    if (slot_stride % gran) return fail(OCO_INVALID_ARGUMENT, "the slot stride must be a multiple of the granularity (%zu bytes)", gran);
    cudaFree(nullptr);   // the runtime's context must exist before the driver calls
    oco_ep_window* w = new oco_ep_window();
    w->rank = rank; w->world = world;
    cudaGetDevice(&w->device);
    w->stride = slot_stride;
    w->backed = (backed_bytes + gran - 1) / gran * gran;
    w->handles.assign(world, 0);
    w->mapped.assign(world, 0);
    CUmemAllocationProp prop = local_prop(w->device);
    CUresult r = drv.reserve(&w->base, w->stride * world, gran, 0, 0);
    if (r != CUDA_SUCCESS) { delete w; return fail(OCO_CUDA_ERROR, "cuMemAddressReserve of %zu bytes failed (%d)", slot_stride * world, (int)r); }
    r = drv.create(&w->handles[rank], w->backed, &prop, 0);
    if (r != CUDA_SUCCESS) {
        drv.address_free(w->base, w->stride * world);
        delete w;
        return fail(OCO_OUT_OF_MEMORY, "cuMemCreate of %zu bytes failed (%d)", backed_bytes, (int)r);
    }
    CUmemAccessDesc access{};
    access.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
    access.location.id = w->device;
    access.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
    const CUdeviceptr mine = w->base + (CUdeviceptr)rank * w->stride;
    r = drv.map(mine, w->backed, 0, w->handles[rank], 0);
    if (r == CUDA_SUCCESS) { w->mapped[rank] = 1; r = drv.set_access(mine, w->backed, &access, 1); }
    if (r == CUDA_SUCCESS) r = drv.export_handle(&w->fd, w->handles[rank], CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0);
    if (r != CUDA_SUCCESS) {
        int code = fail(OCO_CUDA_ERROR, "mapping or exporting the local slot failed (%d)", (int)r);
        oco_ep_window_destroy(w);
        return code;
    }
    *out = w;
    return OCO_OK;
}

int oco_ep_window_fd(const oco_ep_window* w) { return w ? w->fd : -1; }

int oco_ep_window_attach(oco_ep_window* w, int peer, int fd) {
    if (!w || peer < 0 || peer >= w->world || peer == w->rank || fd < 0) return fail(OCO_INVALID_ARGUMENT, "bad peer or descriptor");
    if (w->mapped[peer]) return fail(OCO_INVALID_ARGUMENT, "peer %d is attached already", peer);
    const Driver& drv = driver();
    CUresult r = drv.import_handle(&w->handles[peer], (void*)(uintptr_t)fd, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR);
    if (r != CUDA_SUCCESS) return fail(OCO_CUDA_ERROR, "cuMemImportFromShareableHandle failed (%d)", (int)r);
    const CUdeviceptr at = w->base + (CUdeviceptr)peer * w->stride;
    r = drv.map(at, w->backed, 0, w->handles[peer], 0);
    if (r != CUDA_SUCCESS) {
        drv.release(w->handles[peer]);
        w->handles[peer] = 0;
        return fail(OCO_CUDA_ERROR, "cuMemMap of peer %d's slot failed (%d)", peer, (int)r);
    }
    w->mapped[peer] = 1;
    CUmemAccessDesc access{};
    access.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
    access.location.id = w->device;
    access.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
    r = drv.set_access(at, w->backed, &access, 1);
    if (r != CUDA_SUCCESS) return fail(OCO_CUDA_ERROR, "cuMemSetAccess on peer %d's slot failed (%d): no peer access between the GPUs?", peer, (int)r);
    return OCO_OK;
}

void* oco_ep_window_base(const oco_ep_window* w) { return w ? (void*)w->base : nullptr; }
size_t oco_ep_window_stride(const oco_ep_window* w) { return w ? w->stride : 0; }
size_t oco_ep_window_backed(const oco_ep_window* w) { return w ? w->backed : 0; }

void oco_ep_window_destroy(oco_ep_window* w) {
    if (!w) return;
    const Driver& drv = driver();
    cudaDeviceSynchronize();
    for (int g = 0; g < w->world; g++) {
        if (w->mapped[g]) drv.unmap(w->base + (CUdeviceptr)g * w->stride, w->backed);
        if (w->handles[g]) drv.release(w->handles[g]);
    }
    if (w->base) drv.address_free(w->base, w->stride * w->world);
    if (w->fd >= 0) close(w->fd);
    delete w;
}

}  // extern "C"
