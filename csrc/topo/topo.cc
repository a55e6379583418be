#include "topo.h"
#include <dlfcn.h>
#include <numeric>
#include <sstream>
#include <cuda_runtime.h>
#include "../core/binary_stream.h"
#include "../core/comm.h"
#include "../core/log.h"

namespace hccl {

namespace {
constexpr uint32_t kTopoMagic = 0x544f504fu;  // "TOPO"
constexpr uint32_t kTopoVersion = 2;

void Classify(TopoInfo* t)
{
    t->nServers = (uint32_t)t->serverSizes.size();
    t->symmetric = true;
    uint32_t g = 0;
    for (uint32_t s : t->serverSizes) {
        t->symmetric = t->symmetric && s == t->serverSizes[0];
        g = std::gcd(g, s);
    }
    t->level1Nhr = t->nServers > 1 && g == 1;
    if (t->nRanks == 1) t->level0 = Level0Shape::SINGLE;
}
}  // namespace

std::vector<uint8_t> TopoInfo::Serialize() const
{
    BinaryWriter w;
    w << kTopoMagic << kTopoVersion << nRanks << rank << serverOf << podOf << localOf << nServers << nPods << serverSizes
      << (int32_t)level0 << (int32_t)level0Link << level1Nhr << symmetric << nvls << p2pAll << nvlinkCount << linkGBs
      << deviceName;
    uint64_t h = 1469598103934665603ull;
    for (uint8_t b : w.data()) { h ^= b; h *= 1099511628211ull; }
    w << h;
    return w.Take();
}

bool TopoInfo::Deserialize(const std::vector<uint8_t>& blob, TopoInfo* out)
{
    if (blob.size() < 16) return false;
    uint64_t h = 1469598103934665603ull;
    for (size_t i = 0; i + 8 < blob.size(); ++i) { h ^= blob[i]; h *= 1099511628211ull; }
    BinaryReader r(blob);
    uint32_t magic = 0, ver = 0;
    int32_t l0 = 0, lk = 0;
    TopoInfo t;
    uint64_t stored = 0;
    r >> magic >> ver;
    if (!r.ok() || magic != kTopoMagic || ver != kTopoVersion) return false;
    r >> t.nRanks >> t.rank >> t.serverOf >> t.podOf >> t.localOf >> t.nServers >> t.nPods >> t.serverSizes >> l0 >> lk >>
        t.level1Nhr >> t.symmetric >> t.nvls >> t.p2pAll >> t.nvlinkCount >> t.linkGBs >> t.deviceName >> stored;
    if (!r.ok() || !r.AtEnd() || stored != h) return false;
    // structural guards: vectors must describe exactly nRanks ranks
    if (t.serverOf.size() != t.nRanks || t.podOf.size() != t.nRanks || t.localOf.size() != t.nRanks || t.rank >= t.nRanks) return false;
    if (l0 < 0 || l0 > (int)Level0Shape::SINGLE || lk < 0 || lk > (int)LinkKind::HOST_MEM) return false;
    t.level0 = (Level0Shape)l0;
    t.level0Link = (LinkKind)lk;
    *out = std::move(t);
    return true;
}

std::string TopoInfo::Summary() const
{
    static const char* shapes[] = {"MESH_1D", "CLOS", "MESH_1D_CLOS", "RING", "SINGLE"};
    static const char* links[] = {"none", "NVLink/NVSwitch", "NVLink direct", "PCIe", "network", "host memory"};
    std::ostringstream os;
    os << nRanks << " ranks, " << nServers << " server(s) x " << (serverSizes.empty() ? 0 : serverSizes[0])
       << (symmetric ? "" : " (asymmetric)") << ", " << nPods << " pod(s), level0 " << shapes[(int)level0] << " over "
       << links[(int)level0Link] << ", NVLS " << (nvls ? "yes" : "no") << ", links " << nvlinkCount << ", " << linkGBs
       << " GB/s per direction";
    return os.str();
}

HcclResult BuildTopoFromMeta(const TopoMeta& meta, uint32_t rank, TopoInfo* out)
{
    TopoInfo t;
    uint32_t r = 0, server = 0;
    for (uint32_t pod = 0; pod < meta.size(); ++pod) {
        for (auto& srv : meta[pod]) {
            if (srv.empty()) { HCCL_ERROR("topology literal has an empty server"); return HCCL_E_PARA; }
            for (uint32_t i = 0; i < srv.size(); ++i) {
                t.serverOf.push_back(server);
                t.podOf.push_back(pod);
                t.localOf.push_back(i);
                ++r;
            }
            t.serverSizes.push_back((uint32_t)srv.size());
            ++server;
        }
    }
    if (r == 0 || rank >= r) return HCCL_E_PARA;
    t.nRanks = r;
    t.rank = rank;
    t.nPods = (uint32_t)meta.size();
    t.level0 = Level0Shape::MESH_1D;
    t.level0Link = LinkKind::HOST_MEM;
    t.linkGBs = 10.0;
    Classify(&t);
    *out = std::move(t);
    return HCCL_SUCCESS;
}

namespace {
// NVML is optional: only the number of active NVLink ports is read from it.
uint32_t CountNvlinks(int device)
{
    void* h = dlopen("libnvidia-ml.so.1", RTLD_LAZY | RTLD_LOCAL);
    if (!h) return 0;
    using InitFn = int (*)();
    using GetHandleFn = int (*)(const char*, void**);
    using LinkStateFn = int (*)(void*, unsigned, int*);
    auto init = (InitFn)dlsym(h, "nvmlInit_v2");
    auto shutdown = (InitFn)dlsym(h, "nvmlShutdown");
    auto byPci = (GetHandleFn)dlsym(h, "nvmlDeviceGetHandleByPciBusId_v2");
    auto linkState = (LinkStateFn)dlsym(h, "nvmlDeviceGetNvLinkState");
    uint32_t n = 0;
    if (init && shutdown && byPci && linkState && init() == 0) {
        char pci[32] = {0};
        if (cudaDeviceGetPCIBusId(pci, sizeof(pci), device) == cudaSuccess) {
            void* dev = nullptr;
            if (byPci(pci, &dev) == 0) {
                for (unsigned l = 0; l < 18; ++l) {
                    int active = 0;
                    if (linkState(dev, l, &active) == 0 && active == 1) ++n;
                }
            }
        }
        shutdown();
    }
    dlclose(h);
    return n;
}
}  // namespace

HcclResult DiscoverTopo(CommImpl* comm, TopoInfo* out)
{
    std::vector<uint8_t> blob;
    if (comm->ctx.Get("topo", &blob)) {
        if (TopoInfo::Deserialize(blob, out)) return HCCL_SUCCESS;
        HCCL_WARNING("cached topology failed its integrity check: rediscovering");
        comm->ctx.Erase("topo");
    }
    TopoInfo t;
    t.nRanks = (uint32_t)comm->nRanks;
    t.rank = (uint32_t)comm->rank;
    t.serverOf.assign(t.nRanks, 0);
    t.podOf.assign(t.nRanks, 0);
    t.localOf.resize(t.nRanks);
    for (uint32_t i = 0; i < t.nRanks; ++i) t.localOf[i] = i;
    t.serverSizes = {t.nRanks};
    t.nPods = 1;
    t.level0 = Level0Shape::MESH_1D;
    t.nvls = comm->nvls();
    cudaDeviceProp prop;
    if (cudaGetDeviceProperties(&prop, comm->device) == cudaSuccess) t.deviceName = prop.name;
    if (comm->emulated()) {
        t.level0Link = LinkKind::HOST_MEM;   // all ranks on one GPU: "links" are local memory
        t.linkGBs = 3000.0;
    } else {
        t.nvlinkCount = CountNvlinks(comm->device);
        // With NVLS present or >= 1 active NVLink the box is NVSwitch-connected; 50 GB/s per NVLink-5 port and
        // direction, 18 ports = 900 GB/s.  Without NVLink the peers talk over PCIe.
        if (t.nvls || t.nvlinkCount > 0) {
            t.level0Link = LinkKind::NVLINK_SWITCH;
            t.linkGBs = t.nvlinkCount ? 50.0 * t.nvlinkCount : 900.0;
        } else {
            t.level0Link = LinkKind::PCIE;
            t.linkGBs = 50.0;
        }
    }
    Classify(&t);
    comm->ctx.Put("topo", t.Serialize());
    HCCL_CONFIG_INFO(LOG_MOD_ALG, "comm %s topology: %s", comm->name.c_str(), t.Summary().c_str());
    *out = std::move(t);
    return HCCL_SUCCESS;
}

HcclResult MatchTopo(const TopoInfo& t, TopoMatchKind kind, AlgHierarchy* out)
{
    out->infos.clear();
    auto all = [&] { std::vector<uint32_t> v(t.nRanks); std::iota(v.begin(), v.end(), 0u); return v; };
    if (kind == TopoMatchKind::SQUEEZE_2D) {
        // one physical level (the whole group when it is flat, else not applicable) as a grid
        if (t.nServers > 1) { HCCL_WARNING("squeeze-2D match is for a single physical level"); return HCCL_E_NOT_SUPPORT; }
        uint32_t cols = 1;
        for (uint32_t d = 2; (uint64_t)d * d <= t.nRanks; ++d)
            if (t.nRanks % d == 0) cols = d;
        if (cols == 1) { out->infos.push_back({all()}); return HCCL_SUCCESS; }
        const uint32_t rowLen = t.nRanks / cols;                 // the longer side: consecutive ranks share a row
        std::vector<std::vector<uint32_t>> rows(cols), columns(rowLen);
        for (uint32_t r = 0; r < t.nRanks; ++r) { rows[r / rowLen].push_back(r); columns[r % rowLen].push_back(r); }
        out->infos.push_back(rows);
        out->infos.push_back(columns);
        return HCCL_SUCCESS;
    }
    if (kind == TopoMatchKind::ONE_LEVEL || t.nServers <= 1) {
        out->infos.push_back({all()});
        return HCCL_SUCCESS;
    }
    if (!t.symmetric) {
        HCCL_WARNING("multi-level topology match needs servers of equal size");
        return HCCL_E_NOT_SUPPORT;
    }
    // level 0: one group per server
    std::vector<std::vector<uint32_t>> l0(t.nServers);
    for (uint32_t r = 0; r < t.nRanks; ++r) l0[t.serverOf[r]].push_back(r);
    out->infos.push_back(l0);
    const uint32_t perServer = t.serverSizes[0];
    if (kind == TopoMatchKind::TWO_LEVEL || t.nPods <= 1) {
        // level 1: ranks with the same local index across all servers (a "rail")
        std::vector<std::vector<uint32_t>> l1(perServer);
        for (uint32_t r = 0; r < t.nRanks; ++r) l1[t.localOf[r]].push_back(r);
        out->infos.push_back(l1);
        return HCCL_SUCCESS;
    }
    // three levels: rails inside a pod, then the same (server-in-pod, local) position across pods
    std::vector<uint32_t> serversInPod(t.nPods, 0), firstServer(t.nPods, UINT32_MAX);
    for (uint32_t r = 0; r < t.nRanks; ++r) {
        if (t.localOf[r] == 0) ++serversInPod[t.podOf[r]];
        if (t.serverOf[r] < firstServer[t.podOf[r]]) firstServer[t.podOf[r]] = t.serverOf[r];
    }
    for (uint32_t p = 1; p < t.nPods; ++p)
        if (serversInPod[p] != serversInPod[0]) { HCCL_WARNING("three-level match needs pods of equal size"); return HCCL_E_NOT_SUPPORT; }
    std::vector<std::vector<uint32_t>> l1(t.nPods * perServer), l2(serversInPod[0] * perServer);
    for (uint32_t r = 0; r < t.nRanks; ++r) {
        l1[t.podOf[r] * perServer + t.localOf[r]].push_back(r);
        const uint32_t sInPod = t.serverOf[r] - firstServer[t.podOf[r]];
        l2[sInPod * perServer + t.localOf[r]].push_back(r);
    }
    out->infos.push_back(l1);
    out->infos.push_back(l2);
    return HCCL_SUCCESS;
}

TopoInfo SyntheticNvswitchBox(uint32_t nRanks, bool nvls, double linkGBs)
{
    TopoInfo topo;
    topo.nRanks = nRanks;
    topo.rank = 0;
    topo.serverOf.assign(nRanks, 0);
    topo.podOf.assign(nRanks, 0);
    topo.localOf.resize(nRanks);
    for (uint32_t i = 0; i < nRanks; ++i) topo.localOf[i] = i;
    topo.serverSizes = {nRanks};
    topo.level0 = Level0Shape::MESH_1D;
    topo.level0Link = LinkKind::NVLINK_SWITCH;
    topo.nvls = nvls;
    topo.p2pAll = true;
    topo.nvlinkCount = 18;
    topo.linkGBs = linkGBs;
    topo.deviceName = "NVIDIA B200 (synthetic)";
    return topo;
}

}  // namespace hccl
