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

// Releases whatever a (possibly half-built) VMM segment holds: mappings, address ranges, imported and local handles,
// the multicast binding.  Safe on a segment that is only partly filled in.
void ReleaseVmm(SymSegment* seg, int device)
{
    const DriverApi* d = GetDriverApi();
    if (!d) return;
    if (seg->mc) {
        d->cuMemUnmap((CUdeviceptr)seg->mc, seg->mappedSize);
        d->cuMemAddressFree((CUdeviceptr)seg->mc, seg->mappedSize);
        seg->mc = nullptr;
    }
    if (seg->mcHandle) {
        CUdevice dev;
        // the binding goes before the object: an object released while memory is still bound keeps the switch's
        // multicast group alive until the last bound allocation is freed
        if (seg->mcBound && d->cuMulticastUnbind && d->cuDeviceGet(&dev, device) == CUDA_SUCCESS) d->cuMulticastUnbind(seg->mcHandle, dev, 0, seg->mappedSize);
        d->cuMemRelease(seg->mcHandle);
        seg->mcHandle = 0;
        seg->mcBound = false;
    }
    for (int q = 0; q < seg->nRanks; ++q) {
        if (seg->peer[q]) {
            d->cuMemUnmap((CUdeviceptr)seg->peer[q], seg->mappedSize);
            d->cuMemAddressFree((CUdeviceptr)seg->peer[q], seg->mappedSize);
            seg->peer[q] = nullptr;
        }
        if (q != seg->rank && seg->peerHandle[q]) { d->cuMemRelease(seg->peerHandle[q]); seg->peerHandle[q] = 0; }
    }
    if (seg->localHandle) { d->cuMemRelease(seg->localHandle); seg->localHandle = 0; }
}

// VMM allocation in phases.  Every phase ends in ONE status all ranks agree on: a rank whose local step failed still
// takes part in every exchange of the phase (descriptor passing, barrier, agreement), so the ranks never get out of
// step on the bootstrap, and on an agreed failure every rank releases what it has acquired and returns the same
// error.  Reserved address ranges, imported handles and descriptors are released on every path.
HcclResult AllocVmm(Bootstrap& bs, int device, size_t size, bool wantMc, SymSegment* seg, bool* mcDone)
{
    *mcDone = false;
    const DriverApi* d = GetDriverApi();
    const int p = bs.nRanks(), me = bs.rank();
    bool ok = d != nullptr, all = false;
    // ---- phase 1: create and export the local allocation
    CUdevice dev = 0;
    CUmemAllocationProp prop;
    memset(&prop, 0, sizeof(prop));
    prop.type = CU_MEM_ALLOCATION_TYPE_PINNED;
    prop.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
    prop.location.id = device;
    prop.requestedHandleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
    CUmulticastObjectProp mprop;
    memset(&mprop, 0, sizeof(mprop));
    size_t gran = 0, msize = 0;
    CUmemGenericAllocationHandle h = 0;
    int fd = -1;
    auto step = [&](CUresult r, const char* what) {
        if (ok && r != CUDA_SUCCESS) { HCCL_ERROR("%s failed: %s", what, DriverErrorString(r)); ok = false; }
    };
    if (ok) step(d->cuDeviceGet(&dev, device), "cuDeviceGet");
    if (ok) step(d->cuMemGetAllocationGranularity(&gran, &prop, CU_MEM_ALLOC_GRANULARITY_RECOMMENDED), "cuMemGetAllocationGranularity");
    if (ok && wantMc) {
        mprop.numDevices = (unsigned)p;
        mprop.handleTypes = CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR;
        mprop.size = RoundUp(size, gran);
        size_t mg = 0;
        if (d->cuMulticastGetGranularity(&mg, &mprop, CU_MULTICAST_GRANULARITY_RECOMMENDED) == CUDA_SUCCESS && mg > gran) gran = mg;
    }
    if (ok) {
        msize = RoundUp(size, gran);
        mprop.size = msize;
        step(d->cuMemCreate(&h, msize, &prop, 0), "cuMemCreate");
    }
    if (ok) {
        seg->localHandle = h;
        seg->mappedSize = msize;
        step(d->cuMemExportToShareableHandle(&fd, h, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0), "cuMemExportToShareableHandle");
    }
    CHK_RET(bs.AgreeAll(ok, &all));
    if (!all) {
        if (fd >= 0) ::close(fd);
        ReleaseVmm(seg, device);
        return HCCL_E_DRV;
    }
    // ---- phase 2: pass the descriptors around, import and map every rank's allocation
    HcclResult net = HCCL_SUCCESS;      // a bootstrap failure ends the attempt for everybody (the peers' calls fail too)
    for (int k = 1; k < p && net == HCCL_SUCCESS; ++k) net = bs.SendFd((me + k) % p, fd);
    CUmemAccessDesc acc;
    memset(&acc, 0, sizeof(acc));
    acc.location.type = CU_MEM_LOCATION_TYPE_DEVICE;
    acc.location.id = device;
    acc.flags = CU_MEM_ACCESS_FLAGS_PROT_READWRITE;
    for (int k = 0; k < p && net == HCCL_SUCCESS; ++k) {
        const int q = (me + k) % p;
        CUmemGenericAllocationHandle hq = h;
        if (q != me) {
            int pfd = -1;
            net = bs.RecvFd(q, &pfd);                      // received even after a local failure: the sender has sent it
            if (net != HCCL_SUCCESS) break;
            if (ok) {
                CUresult r = d->cuMemImportFromShareableHandle(&hq, (void*)(uintptr_t)pfd, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR);
                if (r != CUDA_SUCCESS) { HCCL_ERROR("importing rank %d's allocation failed: %s", q, DriverErrorString(r)); ok = false; }
                else seg->peerHandle[q] = hq;
            }
            ::close(pfd);
        }
        if (!ok) continue;
        CUdeviceptr va = 0;
        step(d->cuMemAddressReserve(&va, msize, gran, 0, 0), "cuMemAddressReserve");
        if (!ok) continue;
        CUresult r = d->cuMemMap(va, msize, 0, hq, 0);
        if (r != CUDA_SUCCESS) { d->cuMemAddressFree(va, msize); step(r, "cuMemMap"); continue; }
        seg->peer[q] = (void*)va;                           // from here on ReleaseVmm unmaps and frees the range
        step(d->cuMemSetAccess(va, msize, &acc, 1), "cuMemSetAccess");
    }
    ::close(fd);
    if (net != HCCL_SUCCESS) { ReleaseVmm(seg, device); return net; }
    CHK_RET(bs.AgreeAll(ok, &all));     // also the point after which exporters may drop their descriptors: everyone has imported
    if (!all) { ReleaseVmm(seg, device); return HCCL_E_DRV; }
    if (!wantMc) return HCCL_SUCCESS;
    // ---- phase 3: multicast object, created by rank 0, joined by every device; then each rank binds its allocation.
    // A failure here only turns NVLS off: the peer mappings stay.
    CUmemGenericAllocationHandle mc = 0;
    bool mcOk = true;
    int mfd = -1;
    if (me == 0) {
        CUresult r = d->cuMulticastCreate(&mc, &mprop);
        if (r != CUDA_SUCCESS) { HCCL_WARNING("cuMulticastCreate failed (%s): NVLS off", DriverErrorString(r)); mcOk = false; }
        if (mcOk && d->cuMemExportToShareableHandle(&mfd, mc, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR, 0) != CUDA_SUCCESS) mcOk = false;
    }
    CHK_RET(bs.AgreeAll(mcOk, &all));
    auto dropMc = [&]() {
        if (mfd >= 0) ::close(mfd);
        if (mc) d->cuMemRelease(mc);
    };
    if (!all) { dropMc(); return HCCL_SUCCESS; }
    if (me == 0) {
        for (int q = 1; q < p && net == HCCL_SUCCESS; ++q) net = bs.SendFd(q, mfd);
        ::close(mfd);
        mfd = -1;
    } else {
        net = bs.RecvFd(0, &mfd);
        if (net == HCCL_SUCCESS) {
            if (d->cuMemImportFromShareableHandle(&mc, (void*)(uintptr_t)mfd, CU_MEM_HANDLE_TYPE_POSIX_FILE_DESCRIPTOR) != CUDA_SUCCESS) { mc = 0; mcOk = false; }
            ::close(mfd);
            mfd = -1;
        }
    }
    if (net != HCCL_SUCCESS) { dropMc(); ReleaseVmm(seg, device); return net; }
    if (mcOk && d->cuMulticastAddDevice(mc, dev) != CUDA_SUCCESS) mcOk = false;
    CHK_RET(bs.AgreeAll(mcOk, &all));   // every device must be added before any bind
    if (!all) { dropMc(); return HCCL_SUCCESS; }
    seg->mcHandle = mc;
    CUresult br = d->cuMulticastBindMem(mc, 0, h, 0, msize, 0);
    if (br != CUDA_SUCCESS) { HCCL_WARNING("cuMulticastBindMem failed (%s): NVLS off", DriverErrorString(br)); mcOk = false; }
    else seg->mcBound = true;
    CUdeviceptr mva = 0;
    if (mcOk) {
        if (d->cuMemAddressReserve(&mva, msize, gran, 0, 0) != CUDA_SUCCESS) mcOk = false;
        else if (d->cuMemMap(mva, msize, 0, mc, 0) != CUDA_SUCCESS) { d->cuMemAddressFree(mva, msize); mva = 0; mcOk = false; }
        else {
            seg->mc = (void*)mva;
            if (d->cuMemSetAccess(mva, msize, &acc, 1) != CUDA_SUCCESS) mcOk = false;
        }
    }
    CHK_RET(bs.AgreeAll(mcOk, &all));
    if (!all) {
        // only the multicast part goes: unmap the alias, unbind, release the object
        if (seg->mc) { d->cuMemUnmap((CUdeviceptr)seg->mc, msize); d->cuMemAddressFree((CUdeviceptr)seg->mc, msize); seg->mc = nullptr; }
        if (seg->mcBound) { d->cuMulticastUnbind(mc, dev, 0, msize); seg->mcBound = false; }
        d->cuMemRelease(mc);
        seg->mcHandle = 0;
        return HCCL_SUCCESS;
    }
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
        ReleaseVmm(out, device);      // a rank that succeeded while a peer failed gives its mappings back
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
        int device = 0;
        cudaGetDevice(&device);
        ReleaseVmm(seg, device);      // unmaps the alias, unbinds the allocation from the multicast object, then releases
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
