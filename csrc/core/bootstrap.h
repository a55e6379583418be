// Out-of-band rendezvous between the ranks of one communicator.
//
// HCCL does this in its HCOMM half: HcclGetRootInfo creates a TCP rendezvous
// endpoint on rank 0 whose address travels inside the 4108-byte root info
// (experimental/eco_system/python/PUBLIC_API_en.md:32-33), governed by
// HCCL_IF_IP / HCCL_IF_BASE_PORT / HCCL_CONNECT_TIMEOUT
// (docs/en/user_guide/hccl_env/README.md:26-40).  Here: a star over TCP (a small
// server thread inside the process that created the root info relays
// all-gathers), plus abstract unix datagram sockets to pass file descriptors of
// CUDA VMM allocations between the processes of one box.
#pragma once
#include <cstdint>
#include <deque>
#include <memory>
#include <mutex>
#include <string>
#include <vector>
#include "hccl/hccl_types.h"

namespace hccl {

struct RootInfoPayload {
    uint32_t magic;
    uint32_t version;
    char ip[64];
    uint32_t port;
    uint64_t uniqueId;
};
static_assert(sizeof(RootInfoPayload) <= HCCL_ROOT_INFO_BYTES, "root info payload must fit");
constexpr uint32_t kRootInfoMagic = 0x48434c42u;  // "HCLB"

// Creates the listening endpoint + relay thread and fills `out`.
HcclResult BootstrapCreateRoot(HcclRootInfo* out);
// Index of the interface a rule of HCCL_SOCKET_IFNAME selects among `names` (in that order), -1 for none.
int MatchInterfaceRule(const std::string& rule, const std::vector<std::string>& names);
// Same, with an explicit address (rank-table initialisation); port 0 = ephemeral.
HcclResult BootstrapCreateRootAt(const std::string& ip, uint32_t port, uint64_t uniqueId, HcclRootInfo* out);

class Bootstrap {
public:
    Bootstrap() = default;
    ~Bootstrap();
    Bootstrap(const Bootstrap&) = delete;
    Bootstrap& operator=(const Bootstrap&) = delete;

    HcclResult Connect(const HcclRootInfo& info, int rank, int nRanks, uint32_t timeoutS);
    // recv has nRanks * bytesPerRank bytes; every rank must call with the same size.
    HcclResult AllGather(const void* send, void* recv, size_t bytesPerRank);
    HcclResult Barrier();
    // All ranks obtain the AND of `ok` (used for fallback agreement, reference
    // NegotiateAllReduceMin in comm_negotiation.h:41-50).
    HcclResult AgreeAll(bool ok, bool* all);
    HcclResult SendFd(int peer, int fd);
    HcclResult RecvFd(int peer, int* fd);
    void Close();
    int rank() const { return rank_; }
    int nRanks() const { return nRanks_; }
    uint64_t uniqueId() const { return uniqueId_; }
    // Test hook: when set, the next AllGather fails as if the connection dropped.
    void InjectFailureOnce() { injectFail_ = true; }

private:
    int rank_ = -1, nRanks_ = 0;
    int tcpFd_ = -1;
    int udsFd_ = -1;
    uint64_t uniqueId_ = 0;
    uint32_t timeoutS_ = 120;
    bool injectFail_ = false;
    std::mutex mu_;
    struct PendingFd { int from; int fd; };
    std::deque<PendingFd> pendingFds_;
};

}  // namespace hccl
