// Environment / flag configuration.
//
// Three levels, highest wins: HcclCommConfig > environment > built-in default
// (reference: alg_env_config.h:34-81 for the variable set, :151-187 for the
// getters, op_common.cc:4878-4931 for the per-communicator override).
// Parsing is pure (string -> struct) so that it can be unit-tested without
// touching the process environment.
#pragma once
#include <cstdint>
#include <functional>
#include <utility>
#include <map>
#include <string>
#include <vector>
#include "hccl/hccl_types.h"

namespace hccl {

// Algorithm family names accepted by HCCL_ALGO (reference grammar:
// docs/en/user_guide/hccl_env/HCCL_ALGO.md; parser alg_parse.cc).
enum class AlgoType : int { DEFAULT = 0, NA, RING, HD_R, NHR, NHR_V1, NB, AHC, PIPELINE, PAIRWISE, MESH, ONESHOT, TWOSHOT, NVLS, LL,
                            CONCURRENT, OMNIPIPE, HIER, TREE, DETOUR, SERIAL, TWO_DIE, MESH_CONCUR };   // executor families beyond the reference's HCCL_ALGO names
const char* AlgoTypeName(AlgoType t);
bool ParseAlgoType(const std::string& s, AlgoType* out);

constexpr int kAlgoLevels = 3;
struct AlgoLevelConfig {
    AlgoType level[kAlgoLevels] = {AlgoType::DEFAULT, AlgoType::DEFAULT, AlgoType::DEFAULT};
    bool specified = false;
};
// Result of parsing HCCL_ALGO: a global entry and optional per-op overrides.
struct AlgoConfig {
    AlgoLevelConfig global;
    std::map<HcclCMDType, AlgoLevelConfig> perOp;
    const AlgoLevelConfig& For(HcclCMDType op) const;
};
// Returns false (and fills *err) on a grammar error; mixing the global and the
// per-op form in one string is an error, as in the reference.
bool ParseHcclAlgo(const std::string& value, AlgoConfig* out, std::string* err);

enum class Deterministic : int { OFF = 0, ON = 1, STRICT = 2 };

struct DfsConfig {  // HCCL_DFS_CONFIG
    bool stuckDetection = true;
    bool clusterHeartbeat = true;
    bool inconsistentCheck = true;
    bool taskException = true;
    uint32_t connectionFaultDetectionTimeS = 20;
};

struct EnvConfig {
    AlgoConfig algo;
    HcclCommEngine expansionMode = HCCL_ENGINE_AUTO;  // HCCL_OP_EXPANSION_MODE
    bool planCacheEnable = true;                      // "..._CacheDisable" suffix turns it off
    Deterministic deterministic = Deterministic::OFF; // HCCL_DETERMINISTIC
    uint32_t execTimeoutS = 0;                        // HCCL_EXEC_TIMEOUT, 0 = default
    bool retryL1 = false, retryL2 = false;            // HCCL_OP_RETRY_ENABLE
    uint32_t retryMaxCnt = 1, retryHoldMs = 0, retryIntervalMs = 0; // HCCL_OP_RETRY_PARAMS
    DfsConfig dfs;
    uint32_t debugConfigMask = 0;                     // HCCL_DEBUG_CONFIG
    bool entryLog = false;                            // HCCL_ENTRY_LOG_ENABLE
    bool diagnose = false;                            // HCCL_DIAGNOSE_ENABLE
    uint32_t bufferSizeMiB = 0;                       // HCCL_BUFFSIZE, 0 = default
    std::string ifIp;                                 // HCCL_IF_IP
    uint32_t ifBasePort = 0;                          // HCCL_IF_BASE_PORT
    uint32_t connectTimeoutS = 120;                   // HCCL_CONNECT_TIMEOUT
    std::string socketIfname;                         // HCCL_SOCKET_IFNAME: [^][=]name[,name...] - which NIC gives the rendezvous address
    bool socketIpv6 = false;                          // HCCL_SOCKET_FAMILY=AF_INET6 (the rendezvous speaks IPv4: rejected with a message)
    bool whitelistDisable = true;                     // HCCL_WHITELIST_DISABLE: 0 = only addresses of HCCL_WHITELIST_FILE may join
    std::string whitelistFile;                        // HCCL_WHITELIST_FILE: {"host_ip": ["a.b.c.d", ...]}
    bool hostPortAuto = false;                        // HCCL_HOST_SOCKET_PORT_RANGE=auto
    std::vector<std::pair<uint32_t, uint32_t>> hostPortRanges;   // ... or ports / ranges, first..last inclusive; beats HCCL_IF_BASE_PORT
    std::vector<std::string> notApplicable;           // variables of fabrics this library does not drive (RDMA, PCIe, UB): set, checked, without effect
    std::string tunerPlugin;                          // HCCL_ALG_TUNER_PLUGIN
    std::string algoPlugin;                           // HCCL_ALGO_PLUGIN_PATH
    std::vector<double> splitRatio;                   // HCCL_ALG_MULTIPLE_DIMENSION_SPLIT_RATIO
    bool thresholdSelector = false;                   // HCCL_SELECTOR_MODE=threshold: decision trees instead of the cost model
    std::string algoTree;                             // HCCL_ALGO_TREE: executor tree for the tree-interpreting executor
    // B200-specific knobs
    int nvlsEnable = -1;                              // HCCL_NVLS_ENABLE: -1 auto, 0 off, 1 on
    uint32_t maxBlocks = 0;                           // HCCL_MAX_BLOCKS, 0 = auto
    bool emulate = false;                             // HCCL_B200_EMULATE
    bool forceIpc = false;                            // HCCL_B200_FORCE_IPC: skip VMM, use cudaIpc
    bool a2avLeader = true;                           // HCCL_A2AV_LEADER: AlltoAllV with the size exchange on one block row per rank (0: on every row)
    bool callShapeAgree = true;                       // HCCL_CALL_SHAPE_AGREE: ranks exchange their buffer facts the first time they meet a call signature
    std::vector<std::string> errors;                  // one line per rejected variable
};

// Default device-side wait budget.  HCCL's default is 1836 s
// (HCCL_EXEC_TIMEOUT.md:11-13); on a shared GPU a bounded spin of that length is a
// hang for the next user, so the built-in default here is 30 s and the variable
// can only shorten or lengthen it explicitly.
constexpr uint32_t kDefaultExecTimeoutS = 30;
constexpr uint32_t kDefaultBufferMiB = 256;

using EnvGetter = std::function<const char*(const char*)>;
// Parses every variable through `get` (std::getenv by default).
EnvConfig ParseEnvConfig(const EnvGetter& get);
// Cached process-wide config (parsed on first use); ReloadEnvConfig re-reads.
const EnvConfig& GetEnvConfig();
void ReloadEnvConfig();
uint32_t EnvConfigVersion();     // counts reloads: cached selections are keyed by it (HCCL_ALGO and friends may have changed)

// The effective settings of one communicator after merging HcclCommConfig.
struct EffectiveConfig {
    uint64_t bufferBytes;
    Deterministic deterministic;
    HcclCommEngine engine;
    uint64_t execTimeoutNs;
    uint32_t maxBlocks;
    int nvlsEnable;
    bool planCacheEnable;
    std::string commName;
};
HcclResult MergeConfig(const EnvConfig& env, const HcclCommConfig* cfg, EffectiveConfig* out);

// Timeout chain derived from the exec timeout (reference aicpu_timeout.h:19-58:
// wait = exec, full = +20 s, kernel = +30 s, host-notify = +50 s).
struct TimeoutChain { uint64_t waitNs, fullNs, kernelNs, hostNotifyNs; };
TimeoutChain DeriveTimeouts(uint64_t execTimeoutNs);

}  // namespace hccl
