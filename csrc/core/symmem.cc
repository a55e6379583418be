#include "symmem.h"
#include <cstring>
#include <string>
#include <mutex>
#include <map>
#include <unistd.h>
#include "cuda_driver.h"
#include "log.h"

namespace hccl {

SymCaps QuerySymCaps(int device)
{
    SymCaps caps;
    const DriverApi* d = GetDriverApi();
    if (!d) return caps;
    CUdevice dev;
    if (d->cuDeviceGet(&dev, device) != CUDA_SUCCESS) return caps;
    int v = 0;
    if (d->cuDeviceGetAttribute(&v, CU_DEVICE_ATTRIBUTE_VIRTUAL_MEMORY_MANAGEMENT_SUPPORTED, dev) == CUDA_SUCCESS && v) {
        int fdOk = 0;
        d->cuDeviceGetAttribute(&fdOk, CU_DEVICE_ATTRIBUTE_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR_SUPPORTED, dev);
        caps.vmm = fdOk != 0;
    }
    int mc = 0;
    if (d->cuMulticastCreate && d->cuDeviceGetAttribute(&mc, CU_DEVICE_ATTRIBUTE_MULTICAST_SUPPORTED, dev) == CUDA_SUCCESS)
        caps.multicast = caps.vmm && mc != 0;
    return caps;
}

namespace {

size_t RoundUp(size_t v, size_t g) { return (v + g - 1) / g * g; }

HcclResult AllocVmm(Bootstrap& bs, int device, size_t size, bool wantMc, SymSegment* seg, bool* mcDone)
{
    const DriverApi* d = GetDriverApi();
    if (!d) return HCCL_E_DRV;
    const int p = bs.nRanks(), me = bs.rank();
    CUdevice dev;
    CHK_CU(d->cuDeviceGet(&dev, device));
    CUmemAllocationProp prop;
    memset(&prop, 0, sizeof(prop));
    prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
    prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
    prop.location.id = device;
    prop.requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
    size_t gran = 0;
    CHK_CU(d->cuMemGetAllocationGranularity(&gran, &prop, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED));
    CUmulticastObjectProp mprop;
    memset(&mprop, 0, sizeof(mprop));
    if (wantMc) {
        mprop.numDevices = (unsigned)p;
        mprop.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
        mprop.size = RoundUp(size, gran);
        size_t mg = 0;
        if (d->cuMulticastGetGranularity(&mg, &mprop, CU_MULTICAST_GRANULARITY_RECOMMENDED) == CUDA_SUCCESS && mg > gran) gran = mg;
    }
    const size_t msize = RoundUp(size, gran);
    mprop.size = msize;
    CUmemGenericAllocationHandle h = 0;
    CHK_CU(d->cuMemCreate(&h, msize, &prop, 0));
    seg->localHandle = h;
    seg->mappedSize = msize;
    int fd = -1;
    CHK_CU(d->cuMemExportToShareableHandle(&fd, h, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0));
    for (int k = 1; k < p; ++k) CHK_RET(bs.SendFd((me + k) % p, fd));
    CUmemAccessDesc acc;
    memset(&acc, 0, sizeof(acc));
    acc.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
    acc.location.id = device;
    acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
    for (int k = 0; k < p; ++k) {
        const int q = (me + k) % p;
        CUmemGenericAllocationHandle hq = h;
        if (q != me) {
            int pfd = -1;
            CHK_RET(bs.RecvFd(q, &pfd));
            CUresult r = d->cuMemImportFromShareableHandle(&hq, (void*)(uintptr_t)pfd, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR);
            ::close(pfd);
            if (r != CUDA_SUCCESS) { HCCL_ERROR("importing rank %d's allocation failed: %s", q, DriverErrorString(r)); return HCCL_E_DRV; }
            seg->peerHandle[q] = hq;
        }
        CUdeviceptr va = 0;
        CHK_CU(d->cuMemAddressReserve(&va, msize, gran, 0, 0));
        CHK_CU(d->cuMemMap(va, msize, 0, hq, 0));
        CHK_CU(d->cuMemSetAccess(va, msize, &acc, 1));
        seg->peer[q] = (void*)va;
    }
    ::close(fd);
    CHK_RET(bs.Barrier());  // everyone has imported: exporters may drop their descriptors
    *mcDone = false;
    if (!wantMc) return HCCL_SUCCESS;
    // Multicast object: created by rank 0, joined by every device, then each rank binds its own allocation.
    CUmemGenericAllocationHandle mc = 0;
    bool okLocal = true;
    if (me == 0) {
        CUresult r = d->cuMulticastCreate(&mc, &mprop);
        if (r != CUDA_SUCCESS) { HCCL_WARNING("cuMulticastCreate failed (%s): NVLS off", DriverErrorString(r)); okLocal = false; }
    }
    bool all = false;
    CHK_RET(bs.AgreeAll(okLocal, &all));
    if (!all) return HCCL_SUCCESS;
    if (me == 0) {
        int mfd = -1;
        CHK_CU(d->cuMemExportToShareableHandle(&mfd, mc, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0));
        for (int q = 1; q < p; ++q) CHK_RET(bs.SendFd(q, mfd));
        ::close(mfd);
    } else {
        int mfd = -1;
        CHK_RET(bs.RecvFd(0, &mfd));
        CUresult r = d->cuMemImportFromShareableHandle(&mc, (void*)(uintptr_t)mfd, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR);
        ::close(mfd);
        if (r != CUDA_SUCCESS) okLocal = false;
    }
    if (okLocal && d->cuMulticastAddDevice(mc, dev) != CUDA_SUCCESS) okLocal = false;
    CHK_RET(bs.AgreeAll(okLocal, &all));   // every device must be added before any bind
    if (!all) { if (mc) d->cuMemRelease(mc); return HCCL_SUCCESS; }
    CUresult br = d->cuMulticastBindMem(mc, 0, h, 0, msize, 0);
    if (br != CUDA_SUCCESS) { HCCL_WARNING("cuMulticastBindMem failed (%s): NVLS off", DriverErrorString(br)); okLocal = false; }
    CUdeviceptr mva = 0;
    if (okLocal) {
        if (d->cuMemAddressReserve(&mva, msize, gran, 0, 0) != CUDA_SUCCESS || d->cuMemMap(mva, msize, 0, mc, 0) != CUDA_SUCCESS ||
            d->cuMemSetAccess(mva, msize, &acc, 1) != CUDA_SUCCESS)
            okLocal = false;
    }
    CHK_RET(bs.AgreeAll(okLocal, &all));
    if (!all) {
        if (mva) { d->cuMemUnmap(mva, msize); d->cuMemAddressFree(mva, msize); }
        d->cuMulticastUnbind(mc, dev, 0, msize);
        d->cuMemRelease(mc);
        return HCCL_SUCCESS;
    }
    seg->mc = (void*)mva;
    seg->mcHandle = mc;
    *mcDone = true;
    return HCCL_SUCCESS;
}

HcclResult AllocIpc(Bootstrap& bs, size_t size, SymSegment* seg)
{
    const int p = bs.nRanks(), me = bs.rank();
    void* local = nullptr;
    CHK_CUDA(cudaMalloc(&local, size));
    CHK_CUDA(cudaMemset(local, 0, size));
    cudaIpcMemHandle_t mine;
    CHK_CUDA(cudaIpcGetMemHandle(&mine, local));
    std::vector<cudaIpcMemHandle_t> all((size_t)p);
    CHK_RET(bs.AllGather(&mine, all.data(), sizeof(mine)));
    seg->peer[me] = local;
    for (int q = 0; q < p; ++q) {
        if (q == me) continue;
        void* ptr = nullptr;
        cudaError_t e = cudaIpcOpenMemHandle(&ptr, all[q], cudaIpcMemLazyEnablePeerAccess);
        if (e != cudaSuccess) { HCCL_ERROR("cudaIpcOpenMemHandle for rank %d failed: %s", q, cudaGetErrorString(e)); return HCCL_E_RUNTIME; }
        seg->peer[q] = ptr;
    }
    seg->mappedSize = size;
    return bs.Barrier();
}

}  // namespace

HcclResult SymAlloc(Bootstrap& bs, int device, size_t size, bool wantMc, bool forceIpc, SymSegment* out)
{
    CHK_PTR_NULL(out);
    *out = SymSegment();
    out->size = size;
    out->rank = bs.rank();
    out->nRanks = bs.nRanks();
    if (bs.nRanks() > HCCL_MAX_DEVICE_RANKS) { HCCL_ERROR("at most %d ranks per NVLink domain", HCCL_MAX_DEVICE_RANKS); return HCCL_E_NOT_SUPPORT; }
    SymCaps caps = QuerySymCaps(device);
    bool tryVmm = caps.vmm && !forceIpc, all = false;
    CHK_RET(bs.AgreeAll(tryVmm, &all));
    if (all) {
        bool mcWanted = wantMc && caps.multicast, mcAll = false;
        CHK_RET(bs.AgreeAll(mcWanted, &mcAll));
        bool mcDone = false;
        HcclResult r = AllocVmm(bs, device, size, mcAll, out, &mcDone);
        bool ok = (r == HCCL_SUCCESS), okAll = false;
        // a rank whose VMM path failed half-way cannot take part in the agreement rounds the others
        // are still in, so agreement happens once, after the whole attempt
        if (bs.AgreeAll(ok, &okAll) == HCCL_SUCCESS && okAll) {
            out->transport = SymTransport::VMM;
            CHK_CUDA(cudaMemset(out->peer[out->rank], 0, out->mappedSize));
            CHK_CUDA(cudaDeviceSynchronize());
            return bs.Barrier();
        }
        HCCL_WARNING("VMM symmetric allocation failed on some rank (local result %s): falling back to CUDA IPC", ResultString(r));
        *out = SymSegment();
        out->size = size; out->rank = bs.rank(); out->nRanks = bs.nRanks();
    }
    CHK_RET(AllocIpc(bs, size, out));
    out->transport = SymTransport::IPC;
    return HCCL_SUCCESS;
}

// A process may open an IPC handle only once at a time (two registered buffers often live in the same cudaMalloc
// block of a caching allocator), so open mappings are shared and reference counted.
namespace {
struct IpcMapping { void* base; int refs; };
std::mutex g_ipcMu;
std::map<std::string, IpcMapping> g_ipcOpen;     // key: the 64 handle bytes
std::string HandleKey(const cudaIpcMemHandle_t& h) { return std::string(reinterpret_cast<const char*>(&h), sizeof(h)); }

cudaError_t OpenShared(const cudaIpcMemHandle_t& h, void** base)
{
    std::lock_guard<std::mutex> lk(g_ipcMu);
    auto it = g_ipcOpen.find(HandleKey(h));
    if (it != g_ipcOpen.end()) { ++it->second.refs; *base = it->second.base; return cudaSuccess; }
    cudaError_t e = cudaIpcOpenMemHandle(base, h, cudaIpcMemLazyEnablePeerAccess);
    if (e == cudaSuccess) g_ipcOpen[HandleKey(h)] = IpcMapping{*base, 1};
    return e;
}
void CloseShared(void* base)
{
    std::lock_guard<std::mutex> lk(g_ipcMu);
    for (auto it = g_ipcOpen.begin(); it != g_ipcOpen.end(); ++it) {
        if (it->second.base != base) continue;
        if (--it->second.refs == 0) { cudaIpcCloseMemHandle(base); g_ipcOpen.erase(it); }
        return;
    }
}
}  // namespace

HcclResult SymFree(SymSegment* seg)
{
    if (!seg || seg->transport == SymTransport::NONE) return HCCL_SUCCESS;
    const DriverApi* d = GetDriverApi();
    if (seg->transport == SymTransport::VMM && d) {
        if (seg->mc) {
            d->cuMemUnmap((CUdeviceptr)seg->mc, seg->mappedSize);
            d->cuMemAddressFree((CUdeviceptr)seg->mc, seg->mappedSize);
        }
        if (seg->mcHandle) d->cuMemRelease(seg->mcHandle);
        for (int q = 0; q < seg->nRanks; ++q) {
            if (!seg->peer[q]) continue;
            d->cuMemUnmap((CUdeviceptr)seg->peer[q], seg->mappedSize);
            d->cuMemAddressFree((CUdeviceptr)seg->peer[q], seg->mappedSize);
            if (q != seg->rank && seg->peerHandle[q]) d->cuMemRelease(seg->peerHandle[q]);
        }
        if (seg->localHandle) d->cuMemRelease(seg->localHandle);
    } else if (seg->transport == SymTransport::IPC) {
        for (int q = 0; q < seg->nRanks; ++q) {
            if (!seg->peer[q]) continue;
            if (q == seg->rank) cudaFree(seg->peer[q]);
            else cudaIpcCloseMemHandle(seg->peer[q]);
        }
    } else if (seg->transport == SymTransport::LOCAL) {
        cudaFree(seg->peer[seg->rank]);
    } else if (seg->transport == SymTransport::USER_IPC) {
        for (int q = 0; q < seg->nRanks; ++q)
            if (q != seg->rank && seg->ipcBase[q]) CloseShared(seg->ipcBase[q]);      // the local buffer stays the caller's
    }
    *seg = SymSegment();
    return HCCL_SUCCESS;
}

HcclResult SymRegisterUser(Bootstrap& bs, void* ptr, size_t size, SymSegment* out)
{
    CHK_PTR_NULL(out); CHK_PTR_NULL(ptr);
    *out = SymSegment();
    const int p = bs.nRanks(), me = bs.rank();
    if (p > HCCL_MAX_DEVICE_RANKS) return HCCL_E_NOT_SUPPORT;
    const DriverApi* d = GetDriverApi();
    struct Msg { cudaIpcMemHandle_t handle; uint64_t offset, size; int ok; } mine;
    memset(&mine, 0, sizeof(mine));
    mine.size = size;
    CUdeviceptr base = 0;
    size_t range = 0;
    // an IPC handle names a whole allocation: ship the offset of the buffer inside it as well
    if (d != nullptr && d->cuMemGetAddressRange(&base, &range, (CUdeviceptr)ptr) == CUDA_SUCCESS && (char*)ptr + size <= (char*)base + range &&
        cudaIpcGetMemHandle(&mine.handle, (void*)base) == cudaSuccess) {
        mine.offset = (uint64_t)((char*)ptr - (char*)base);
        mine.ok = 1;
    } else {
        cudaGetLastError();
    }
    std::vector<Msg> all((size_t)p);
    CHK_RET(bs.AllGather(&mine, all.data(), sizeof(mine)));
    for (const Msg& m : all) {
        if (!m.ok) { HCCL_ERROR("buffer registration: a rank passed memory that cannot be shared through CUDA IPC (not a cudaMalloc allocation?)"); return HCCL_E_PARA; }
        if (m.size != size) { HCCL_ERROR("buffer registration: ranks passed different sizes (%llu vs %llu)", (unsigned long long)size, (unsigned long long)m.size); return HCCL_E_PARA; }
    }
    out->size = out->mappedSize = size;
    out->rank = me;
    out->nRanks = p;
    out->transport = SymTransport::USER_IPC;
    out->peer[me] = ptr;
    bool ok = true;
    for (int q = 0; q < p; ++q) {
        if (q == me) continue;
        void* mapped = nullptr;
        cudaError_t e = OpenShared(all[(size_t)q].handle, &mapped);
        if (e != cudaSuccess) { HCCL_ERROR("cudaIpcOpenMemHandle for rank %d failed: %s", q, cudaGetErrorString(e)); cudaGetLastError(); ok = false; continue; }
        out->ipcBase[q] = mapped;
        out->peer[q] = (char*)mapped + all[(size_t)q].offset;
    }
    bool allOk = false;
    CHK_RET(bs.AgreeAll(ok, &allOk));
    if (!allOk) { SymFree(out); return HCCL_E_RUNTIME; }
    return HCCL_SUCCESS;
}

HcclResult SymAllocLocalGroup(int nRanks, size_t size, std::vector<SymSegment>* out)
{
    out->assign((size_t)nRanks, SymSegment());
    std::vector<void*> ptrs((size_t)nRanks, nullptr);
    for (int r = 0; r < nRanks; ++r) {
        CHK_CUDA(cudaMalloc(&ptrs[r], size));
        CHK_CUDA(cudaMemset(ptrs[r], 0, size));
    }
    for (int r = 0; r < nRanks; ++r) {
        SymSegment& s = (*out)[r];
        s.size = size; s.mappedSize = size; s.transport = SymTransport::LOCAL; s.rank = r; s.nRanks = nRanks;
        for (int q = 0; q < nRanks; ++q) s.peer[q] = ptrs[q];
    }
    return HCCL_SUCCESS;
}

}  // namespace hccl
