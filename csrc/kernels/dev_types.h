// Plain-C++ types shared by host code and device code: the device view of a
// communicator, the host-visible status block, slab layout constants and the
// argument blocks of the collective kernels.  No device code in this header.
#pragma once
#include <stddef.h>
#include <stdint.h>

namespace hccl {

constexpr int kMaxDevRanks = 8;
constexpr int kMaxBlocks = 128;     // block rows with private flags / epochs
constexpr int kFlagSlots = 4;       // independent signal channels per block row
constexpr int kFlagStride = 1;      // in uint64_t
// Flag area layout per rank: [kMaxBlocks][kFlagSlots][kMaxDevRanks] uint64_t.
constexpr size_t kFlagWords = (size_t)kMaxBlocks * kFlagSlots * kMaxDevRanks;
constexpr size_t kFlagBytes = kFlagWords * sizeof(uint64_t);   // 32 KiB
// LL (flag-in-data) region: 2 parities x kMaxDevRanks slots x kLLSlotBytes.
constexpr size_t kLLMaxPayload = 256 * 1024;            // bytes of payload per rank and op
constexpr size_t kLLSlotBytes = 2 * kLLMaxPayload;      // 8 B data + 8 B flag per 16 B line
constexpr size_t kLLRegionBytes = 2 * kMaxDevRanks * kLLSlotBytes;  // 8 MiB
// Offsets inside a rank's symmetric slab.
constexpr size_t kSlabFlagsOff = 0;
constexpr size_t kSlabP2pFlagsOff = kFlagBytes;                       // send/recv mailbox flags
constexpr size_t kP2pFlagBytes = 64 * 1024;
constexpr size_t kSlabLLOff = 128 * 1024;
constexpr size_t kSlabDataOff = kSlabLLOff + kLLRegionBytes;          // staging starts here (2 MiB aligned by construction)

enum KernelId : uint32_t {
    K_BARRIER = 1, K_AR_LL, K_AR_ONESHOT, K_AR_TWOSHOT, K_AR_NVLS, K_RS, K_RS_NVLS, K_RS_LL, K_AG, K_AG_NVLS, K_AG_LL,
    K_BCAST, K_BCAST_NVLS, K_REDUCE, K_SCATTER, K_A2A, K_A2AV, K_SENDRECV, K_MOE_DISPATCH, K_MOE_COMBINE,
    K_MC2_AG_GEMM, K_MC2_GEMM_RS, K_MC2_GEMM_AR, K_TEST_WAIT
};
enum DevErr : uint32_t { DEV_OK = 0, DEV_ERR_TIMEOUT = 1, DEV_ERR_BOUNDS = 2, DEV_ERR_ABORTED = 3 };

// Host-mapped (pinned, zero-copy) status block, one per communicator.
struct DevStatus {
    volatile uint32_t error;      // DevErr of the first failure
    volatile uint32_t kernelId;   // which kernel family reported
    volatile uint32_t block;      // block row
    volatile uint32_t slot;       // flag slot
    volatile uint32_t peer;       // rank that was expected to signal
    volatile uint32_t rank;       // reporting rank
    volatile uint64_t expected;   // flag value waited for
    volatile uint64_t seen;       // last value observed
    volatile uint64_t head;       // ops started  (stuck detection: head != tail for long = hung op)
    volatile uint64_t tail;       // ops finished
};

struct DevComm {
    int rank;
    int nRanks;
    char* slab[kMaxDevRanks];       // every rank's symmetric slab mapped in this address space
    char* slabMc;                   // multicast alias of the slab (NVLS) or nullptr
    uint64_t* epochs;               // local: [kMaxBlocks] barrier epochs | [kMaxBlocks] LL op counters | head, tail
    uint32_t* abortWord;            // local: non-zero once any wait on this rank gave up
    DevStatus* status;              // host-mapped
    uint64_t timeoutNs;             // budget of one wait
    uint64_t stageBytes;            // usable staging bytes (after kSlabDataOff)
};

constexpr size_t kEpochWords = 2 * kMaxBlocks + 8;
// AlltoAll table at the start of the exchange region: per block row, every peer's send displacement and send size
constexpr size_t kA2aMetaBytes = (size_t)kMaxBlocks * 2 * kMaxDevRanks * sizeof(uint64_t);

enum CollMode : uint32_t {
    MODE_STAGE_IN = 1u,    // copy local `in` into own slab (args.src[rank]) before the first barrier
    MODE_STAGE_OUT = 2u,   // results land in the slab first and are copied to `out` at the end
    MODE_PUSH = 4u,        // args.dst[] are peer-visible outputs: write results to every rank directly
    MODE_INPLACE = 8u,
};

struct CollArgs {
    const char* in;                      // local user input
    char* out;                           // local user output
    const char* src[kMaxDevRanks];       // where this rank reads rank r's input from
    char* dst[kMaxDevRanks];             // MODE_PUSH: where this rank writes rank r's output
    char* xch[kMaxDevRanks];             // exchange region in rank r's slab (phase-2 pull source)
    const char* srcMc;                   // multicast alias of src (NVLS)
    char* dstMc;                         // multicast alias of dst / xch (NVLS)
    uint64_t bytes;                      // payload bytes (meaning per op, see bodies)
    uint64_t cnt[kMaxDevRanks];          // V variants: bytes per rank
    uint64_t dsp[kMaxDevRanks];          // V variants: byte displacement per rank
    uint64_t cnt2[kMaxDevRanks];
    uint64_t dsp2[kMaxDevRanks];
    int op;
    int root;
    uint32_t mode;
    uint32_t pad;
    uint64_t chunk;                      // AlltoAllV staged through the slab: bytes of one pair's staging window (0: one pass)
    float scale;                         // reductions: factor applied to the reduced value before it is stored (1 = none)
    int outType;                         // reductions: HcclDataType of `out` when it differs from the input type, else -1
};

struct P2pItem {
    char* buf;
    uint64_t bytes;
    int peer;
    int isSend;
};
constexpr int kMaxP2pItems = 64;
struct P2pArgs {
    P2pItem items[kMaxP2pItems];
    int nItems;
    uint64_t halfBytes;                  // size of one mailbox half
    uint64_t mailboxOff;                 // offset of the mailbox area inside the slab data region
    uint64_t* seq;                       // local: [2][kMaxDevRanks] next chunk number (send row, recv row)
};

}  // namespace hccl
