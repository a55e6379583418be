// Public scalar types, enums and POD structs of the hccl_b200 C API.
//
// The enum values follow the published HCCL ABI (reference: the value list in
// src/common/hccl_common.h:50-67 and the "gap at 13" rule in
// src/common/hccl_common.h:60-75), so binaries and ctypes bindings written
// against HCCL keep their numeric constants.  Streams are CUDA streams.
#ifndef HCCL_B200_TYPES_H_
#define HCCL_B200_TYPES_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef enum {
    HCCL_SUCCESS = 0,
    HCCL_E_PARA = 1,
    HCCL_E_PTR = 2,
    HCCL_E_MEMORY = 3,
    HCCL_E_INTERNAL = 4,
    HCCL_E_NOT_SUPPORT = 5,
    HCCL_E_NOT_FOUND = 6,
    HCCL_E_UNAVAIL = 7,
    HCCL_E_SYSCALL = 8,
    HCCL_E_TIMEOUT = 9,
    HCCL_E_OPEN_FILE_FAILURE = 10,
    HCCL_E_TCP_CONNECT = 11,
    HCCL_E_ROCE_CONNECT = 12,
    HCCL_E_TCP_TRANSFER = 13,
    HCCL_E_ROCE_TRANSFER = 14,
    HCCL_E_RUNTIME = 15,
    HCCL_E_DRV = 16,
    HCCL_E_PROFILING = 17,
    HCCL_E_CCE = 18,
    HCCL_E_NETWORK = 19,
    HCCL_E_AGAIN = 20,
    HCCL_E_REMOTE = 21,
    HCCL_E_SUSPENDING = 22,
    HCCL_E_OPRETRY_FAIL = 23,
    HCCL_E_OOM = 24,
    HCCL_E_RESERVED
} HcclResult;

typedef enum {
    HCCL_REDUCE_SUM = 0,
    HCCL_REDUCE_PROD = 1,
    HCCL_REDUCE_MAX = 2,
    HCCL_REDUCE_MIN = 3,
    HCCL_REDUCE_RESERVED
} HcclReduceOp;

typedef enum {
    HCCL_DATA_TYPE_INT8 = 0,
    HCCL_DATA_TYPE_INT16 = 1,
    HCCL_DATA_TYPE_INT32 = 2,
    HCCL_DATA_TYPE_FP16 = 3,
    HCCL_DATA_TYPE_FP32 = 4,
    HCCL_DATA_TYPE_INT64 = 5,
    HCCL_DATA_TYPE_UINT64 = 6,
    HCCL_DATA_TYPE_UINT8 = 7,
    HCCL_DATA_TYPE_UINT16 = 8,
    HCCL_DATA_TYPE_UINT32 = 9,
    HCCL_DATA_TYPE_FP64 = 10,
    HCCL_DATA_TYPE_BFP16 = 11,
    HCCL_DATA_TYPE_INT128 = 12,
    /* 13 is a reserved gap and is never valid */
    HCCL_DATA_TYPE_HIF8 = 14,
    HCCL_DATA_TYPE_FP8E4M3 = 15,
    HCCL_DATA_TYPE_FP8E5M2 = 16,
    HCCL_DATA_TYPE_FP8E8M0 = 17,
    HCCL_DATA_TYPE_RESERVED = 255
} HcclDataType;

// Operation identifiers; used by the selector, the tuner ABI and the MC2 API.
typedef enum {
    HCCL_CMD_INVALID = 0,
    HCCL_CMD_BROADCAST = 1,
    HCCL_CMD_ALLREDUCE = 2,
    HCCL_CMD_REDUCE = 3,
    HCCL_CMD_SEND = 4,
    HCCL_CMD_RECEIVE = 5,
    HCCL_CMD_ALLGATHER = 6,
    HCCL_CMD_REDUCE_SCATTER = 7,
    HCCL_CMD_ALLTOALLV = 8,
    HCCL_CMD_ALLTOALLVC = 9,
    HCCL_CMD_ALLTOALL = 10,
    HCCL_CMD_GATHER = 11,
    HCCL_CMD_SCATTER = 12,
    HCCL_CMD_BATCH_SEND_RECV = 13,
    HCCL_CMD_BATCH_PUT = 14,
    HCCL_CMD_BATCH_GET = 15,
    HCCL_CMD_ALLGATHER_V = 16,
    HCCL_CMD_REDUCE_SCATTER_V = 17,
    HCCL_CMD_BARRIER = 18,
    HCCL_CMD_MAX
} HcclCMDType;

typedef enum {
    HCCL_SEND = 0,
    HCCL_RECV = 1,
    HCCL_SEND_RECV_RESERVED
} HcclSendRecvType;

typedef struct {
    HcclSendRecvType sendRecvType;
    void* buf;
    uint64_t count;
    HcclDataType dataType;
    uint32_t remoteRank;
} HcclSendRecvItem;

// Communicator status as seen by HcclCommGetStatus.
typedef enum {
    HCCL_COMM_STATUS_READY = 0,
    HCCL_COMM_STATUS_SUSPENDING = 1,
    HCCL_COMM_STATUS_ERROR = 2,
    HCCL_COMM_STATUS_DESTROYED = 3
} HcclCommStatus;

// Execution engines of this library (the analogue of HCCL's
// AICPU / AIV / CCU / HOSTCPU expansion modes, re-cut for one NVSwitch box).
typedef enum {
    HCCL_ENGINE_AUTO = 0,
    HCCL_ENGINE_P2P = 1,   // SM kernels using peer loads/stores over NVLink
    HCCL_ENGINE_NVLS = 2,  // SM kernels using multimem.* through the NVSwitch
    HCCL_ENGINE_HOSTCPU = 3, // host threads on host memory (simulated ranks)
    HCCL_ENGINE_MAX
} HcclCommEngine;

#define HCCL_ROOT_INFO_BYTES 4108
#define HCCL_COMM_CONFIG_NAME_MAX 128
#define HCCL_MAX_DEVICE_RANKS 8

typedef struct {
    char internal[HCCL_ROOT_INFO_BYTES];
} HcclRootInfo;

// Per-communicator configuration (highest priority; then environment, then
// defaults).  Initialise with HcclCommConfigInit before filling fields.
typedef struct {
    uint32_t size;          // sizeof(HcclCommConfig), set by HcclCommConfigInit
    uint32_t magicWord;
    uint32_t version;
    uint32_t reserved;
    uint32_t hcclBufferSize;    // staging slab in MiB; 0 = HCCL_BUFFSIZE / default
    uint32_t hcclDeterministic; // 0 off, 1 on, 2 strict; 0xFFFFFFFF = unset
    char hcclCommName[HCCL_COMM_CONFIG_NAME_MAX];
    uint32_t hcclOpExpansionMode; // HcclCommEngine; 0 = auto
    uint32_t hcclExecTimeoutMs;   // device wait budget; 0 = env / default
    uint32_t hcclMaxBlocks;       // 0 = auto
    uint32_t hcclNvlsEnable;      // 0 = auto, 1 = force off, 2 = force on
    char padding[2304 - 16 - 4 * 2 - HCCL_COMM_CONFIG_NAME_MAX - 4 * 4];
} HcclCommConfig;

#define HCCL_COMM_CONFIG_MAGIC 0xf0f0f0f0u
#define HCCL_COMM_CONFIG_VERSION 1u
#define HCCL_COMM_CONFIG_UNSET 0xFFFFFFFFu

static inline void HcclCommConfigInit(HcclCommConfig* cfg)
{
    if (cfg == NULL) return;
    char* p = (char*)cfg;
    for (size_t i = 0; i < sizeof(HcclCommConfig); ++i) p[i] = 0;
    cfg->size = (uint32_t)sizeof(HcclCommConfig);
    cfg->magicWord = HCCL_COMM_CONFIG_MAGIC;
    cfg->version = HCCL_COMM_CONFIG_VERSION;
    cfg->hcclDeterministic = HCCL_COMM_CONFIG_UNSET;
}

typedef void* HcclComm;
// A CUDA stream handle (cudaStream_t); kept opaque so that this header needs
// no CUDA include.
typedef void* hcclStream_t;

#ifdef __cplusplus
}
#endif
#endif  // HCCL_B200_TYPES_H_
