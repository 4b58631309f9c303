// Peer-visible device memory from the virtual-memory-management API: physical memory created with
// cuMemCreate, mapped with 2 MiB pages here and - through a POSIX file descriptor passed over a Unix
// socket - in every other process of the machine.
//
// Why not the 64-byte cudaIpc handles alone: a kernel that streams stores into several peers'
// matrices touches hundreds of megabytes of each mapping at once.  Into cudaIpcOpenMemHandle
// mappings the N-sharded W8A8 GEMM's epilogue push reached 310 GB/s per GPU on 4 B200s (2.25 ms
// for 8192 x 28672 fp32); into mappings made by this file the same kernel reaches 640 GB/s (1.10 ms;
// 1.25 ms on 8 GPUs), close to the 680 GB/s of a bare store kernel between GPUs of one process.  The
// handle-based calls stay for small exchange buffers and as the fallback where file descriptors
// cannot be passed.
//
// The driver entry points are resolved through the runtime, as for the tensor maps, so the
// library carries no link-time dependency on libcuda.
#include <cuda.h>
#include <unistd.h>

#include <mutex>
#include <string>

#include "common.cuh"

namespace lhb {
namespace {

struct Vmm {
    CUresult (*create)(CUmemGenericAllocationHandle*, size_t, const CUmemAllocationProp*, unsigned long long) = nullptr;
    CUresult (*release)(CUmemGenericAllocationHandle) = nullptr;
    CUresult (*granularity)(size_t*, const CUmemAllocationProp*, CUmemAllocationGranularity_flags) = nullptr;
    CUresult (*reserve)(CUdeviceptr*, size_t, size_t, CUdeviceptr, unsigned long long) = nullptr;
    CUresult (*addr_free)(CUdeviceptr, size_t) = nullptr;
    CUresult (*map)(CUdeviceptr, size_t, size_t, CUmemGenericAllocationHandle, unsigned long long) = nullptr;
    CUresult (*unmap)(CUdeviceptr, size_t) = nullptr;
    CUresult (*set_access)(CUdeviceptr, size_t, const CUmemAccessDesc*, size_t) = nullptr;
    CUresult (*export_handle)(void*, CUmemGenericAllocationHandle, CUmemAllocationHandleType, unsigned long long) = nullptr;
    CUresult (*import_handle)(CUmemGenericAllocationHandle*, void*, CUmemAllocationHandleType) = nullptr;
    bool ok = false;
};

template <typename F>
bool resolve(const char* name, F* fn) {
    void* p = nullptr;
    cudaDriverEntryPointQueryResult q;
    if (cudaGetDriverEntryPoint(name, &p, cudaEnableDefault, &q) != cudaSuccess || q != cudaDriverEntryPointSuccess || !p) {
        cudaGetLastError();
        return false;
    }
    *fn = reinterpret_cast<F>(p);
    return true;
}

const Vmm& vmm() {
    static Vmm v;
    static std::once_flag once;
    std::call_once(once, [] {
        v.ok = resolve("cuMemCreate", &v.create) && resolve("cuMemRelease", &v.release) &&
               resolve("cuMemGetAllocationGranularity", &v.granularity) && resolve("cuMemAddressReserve", &v.reserve) &&
               resolve("cuMemAddressFree", &v.addr_free) && resolve("cuMemMap", &v.map) && resolve("cuMemUnmap", &v.unmap) &&
               resolve("cuMemSetAccess", &v.set_access) && resolve("cuMemExportToShareableHandle", &v.export_handle) &&
               resolve("cuMemImportFromShareableHandle", &v.import_handle);
    });
    return v;
}

int fail(const char* what, CUresult r) {
    set_last_error_text(std::string(what) + " failed with CUresult " + std::to_string(static_cast<int>(r)));
    return LHB_ERR_CUDA;
}

CUmemAllocationProp prop_for(int device) {
    CUmemAllocationProp prop = {};
    prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
    prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
    prop.location.id = device;
    prop.requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
    return prop;
}

// reserve a range, map `h` into it and open it for reads and writes from `device`
int map_for(const Vmm& v, CUmemGenericAllocationHandle h, size_t bytes, size_t gran, int device, void** out) {
    CUdeviceptr va = 0;
    CUresult r = v.reserve(&va, bytes, gran, 0, 0);
    if (r != CUDA_SUCCESS) return fail("cuMemAddressReserve", r);
    r = v.map(va, bytes, 0, h, 0);
    if (r != CUDA_SUCCESS) { v.addr_free(va, bytes); return fail("cuMemMap", r); }
    CUmemAccessDesc acc = {};
    acc.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
    acc.location.id = device;
    acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
    r = v.set_access(va, bytes, &acc, 1);
    if (r != CUDA_SUCCESS) { v.unmap(va, bytes); v.addr_free(va, bytes); return fail("cuMemSetAccess", r); }
    *out = reinterpret_cast<void*>(va);
    return LHB_OK;
}

}  // namespace
}  // namespace lhb

using namespace lhb;

extern "C" {

int lhb_peer_alloc_shareable(void** out, size_t bytes, int* fd_out, size_t* mapped_bytes) {
    if (!out || !fd_out || !mapped_bytes) return LHB_ERR_NULL;
    if (bytes == 0) return LHB_ERR_BAD_SHAPE;
    *out = nullptr; *fd_out = -1; *mapped_bytes = 0;
    int device = 0;
    LHB_CUDA(cudaGetDevice(&device));
    LHB_CUDA(cudaFree(nullptr));                               // the primary context exists before driver calls
    const Vmm& v = vmm();
    if (!v.ok) { set_last_error_text("the driver's virtual memory management entry points are unavailable"); return LHB_ERR_UNSUPPORTED; }
    const CUmemAllocationProp prop = prop_for(device);
    size_t gran = 0;
    CUresult r = v.granularity(&gran, &prop, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED);
    if (r != CUDA_SUCCESS || gran == 0) return fail("cuMemGetAllocationGranularity", r);
    const size_t padded = (bytes + gran - 1) / gran * gran;
    CUmemGenericAllocationHandle h = 0;
    r = v.create(&h, padded, &prop, 0);
    if (r != CUDA_SUCCESS) return fail("cuMemCreate", r);
    int fd = -1;
    r = v.export_handle(&fd, h, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0);
    if (r != CUDA_SUCCESS) { v.release(h); return fail("cuMemExportToShareableHandle", r); }
    void* p = nullptr;
    const int e = map_for(v, h, padded, gran, device, &p);
    v.release(h);                                              // the mapping (and the descriptor) keep the memory alive
    if (e != LHB_OK) { ::close(fd); return e; }
    cudaError_t ce = cudaMemset(p, 0, padded);
    if (ce == cudaSuccess) ce = cudaDeviceSynchronize();
    if (ce != cudaSuccess) {
        set_last_error("cudaMemset(shareable peer buffer)", ce);
        v.unmap(reinterpret_cast<CUdeviceptr>(p), padded);
        v.addr_free(reinterpret_cast<CUdeviceptr>(p), padded);
        ::close(fd);
        return LHB_ERR_CUDA;
    }
    *out = p; *fd_out = fd; *mapped_bytes = padded;
    return LHB_OK;
}

int lhb_peer_open_fd(int fd, size_t mapped_bytes, void** out) {
    if (!out) return LHB_ERR_NULL;
    if (fd < 0 || mapped_bytes == 0) return LHB_ERR_BAD_SHAPE;
    *out = nullptr;
    int device = 0;
    LHB_CUDA(cudaGetDevice(&device));
    LHB_CUDA(cudaFree(nullptr));
    const Vmm& v = vmm();
    if (!v.ok) { set_last_error_text("the driver's virtual memory management entry points are unavailable"); return LHB_ERR_UNSUPPORTED; }
    const CUmemAllocationProp prop = prop_for(device);
    size_t gran = 0;
    CUresult r = v.granularity(&gran, &prop, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED);
    if (r != CUDA_SUCCESS || gran == 0) return fail("cuMemGetAllocationGranularity", r);
    if (mapped_bytes % gran) return LHB_ERR_BAD_SHAPE;
    CUmemGenericAllocationHandle h = 0;
    r = v.import_handle(&h, reinterpret_cast<void*>(static_cast<intptr_t>(fd)), CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR);
    if (r != CUDA_SUCCESS) return fail("cuMemImportFromShareableHandle", r);
    const int e = map_for(v, h, mapped_bytes, gran, device, out);
    v.release(h);
    return e;
}

int lhb_peer_unmap(void* ptr, size_t mapped_bytes) {
    if (!ptr) return LHB_OK;
    const Vmm& v = vmm();
    if (!v.ok) return LHB_ERR_UNSUPPORTED;
    CUresult r = v.unmap(reinterpret_cast<CUdeviceptr>(ptr), mapped_bytes);
    if (r != CUDA_SUCCESS) return fail("cuMemUnmap", r);
    r = v.addr_free(reinterpret_cast<CUdeviceptr>(ptr), mapped_bytes);
    if (r != CUDA_SUCCESS) return fail("cuMemAddressFree", r);
    return LHB_OK;
}

}  // extern "C"
