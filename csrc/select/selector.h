// Algorithm registry, attributes, cost model, cost table and selection.
//
// Reference structure (src/ops/op_common/selector/):
//   * registry: REGISTER_EXEC_V2 keys a factory by (op, algName) and appends
//     (algName, executor, templates) to the global list
//     (coll_alg_v2_exec_registry.h:34-176, cost_model.cc:48-81);
//   * attributes: REGISTER_ALG_ATTRS(name, topo.*, op.*) (alg_attrs.h:45-111);
//   * cost model per communicator: InitModel -> FilterByEngine ->
//     ApplyHcclAlgoPriority -> FilterByTopoAndCalibrate -> ApplyTopoPriority
//     (cost_model.cc:314-325), coefficients {A,B,C,D} per segment (:443);
//   * cost table per call: cost = sum_groups agg((A/util + B + Bre) * size + C),
//     floored by sum D (cost_table.cc:360-434), util from measured
//     link-utilisation-vs-size tables (:437-457);
//   * engine: tuner may rewrite costs, then min cost inside the best engine tier,
//     ties -> first registered (selector_engine.cc:413-482, :693-704); on failure
//     a per-algorithm trace says which filter removed it (:241-310).
// Retargeted: link parameters are measured NVLink 5 / NVSwitch figures per
// message size (tables in cost_tables.cc) instead of HCCS / RoCE constants.
#pragma once
#include <cstdint>
#include <functional>
#include <map>
#include <memory>
#include <string>
#include <vector>
#include "../core/config.h"
#include "../topo/topo.h"
#include "hccl/hccl_tuner_plugin.h"
#include "hccl/hccl_types.h"

namespace hccl {

class CommImpl;

// What one call looks like to the selector.
struct OpDesc {
    HcclCMDType op = HCCL_CMD_INVALID;
    HcclDataType dtype = HCCL_DATA_TYPE_RESERVED;
    HcclReduceOp redOp = HCCL_REDUCE_RESERVED;
    uint64_t bytes = 0;          // payload the cost scales with (AllReduce: message; AG/RS: per-rank block * p)
    uint32_t root = 0;
    uint32_t nRanks = 1;
    bool inRegistered = false;   // input lies in symmetric memory (peers can read it in place)
    bool outRegistered = false;
    bool inMulticast = false;    // ... and has a multicast alias (switch reductions can read it in place)
    bool outMulticast = false;
    bool aligned16 = true;       // both pointers 16-byte aligned
    bool inPlace = false;
    bool isMc2 = false;          // called on behalf of a fused matmul kernel
    uint64_t stageInBytes = 0;   // size of the communicator's stage-in region (forms that land data there check their fit)
    bool castScale = false;      // the reduction casts to another type and / or scales: only the cast forms can run it
    Deterministic det = Deterministic::OFF;
    HcclCommEngine engine = HCCL_ENGINE_AUTO;   // requested engine (HCCL_OP_EXPANSION_MODE / comm config)
    uint32_t Flags() const;
    // What all ranks can rely on when their local flag words are `a` and `b` (associative, commutative): registration,
    // multicast and alignment only if both have them, in place if either works in place.
    static uint32_t CombineFlags(uint32_t a, uint32_t b);
    void ApplyFlags(uint32_t flags);    // overwrites the per-buffer facts with those of a (combined) flag word
};

enum class NetType : int { LOCAL = 0, MESH_P2P = 1, NVLS_SWITCH = 2, HOST_MEM = 3 };
enum class CostAgg : int { SUM = 0, MAX = 1 };   // Concurrent executors aggregate with MAX (executor_v2_base.h:130-141)

// One segment of the cost formula.  Times in microseconds, sizes in bytes.
struct CostCoeff {
    double A = 0;      // link time per byte at utilisation 1  (us/B)
    double B = 0;      // local copy time per byte             (us/B)
    double Bre = 0;    // local reduce time per byte           (us/B)
    double C = 0;      // fixed latency                        (us)
    double D = 0;      // floor                                (us)
    NetType net = NetType::MESH_P2P;
    double ratio = 1;  // fraction of the message that this segment moves per link (utilisation lookup key)
    int group = 0;
};

struct AlgAttrs {
    uint32_t minLevels = 1, maxLevels = 1;
    bool enforceMaxLevels = false;           // true: not usable on a topology with more levels than maxLevels
    uint32_t level0Shapes = 0xFFFFFFFFu;     // bitmask over Level0Shape
    uint32_t maxRankSize = 0;                // 0 = unlimited
    uint32_t minRankSize = 1;
    bool powerOfTwoRanksOnly = false;
    uint64_t dtypeMask = ~0ull;              // bit (1 << HcclDataType)
    bool supportProd = true;
    bool supportMaxMin = true;
    bool supportInplace = true;
    bool orderPreserved = true;              // fixed reduction order (usable under HCCL_DETERMINISTIC=strict)
    bool deterministic = true;               // run-to-run reproducible
    bool needsNvls = false;
    bool needsDeviceP2p = false;
    bool needsAligned16 = false;
    bool needsRegisteredOut = false;
    uint64_t minBytes = 0, maxBytes = ~0ull;
    bool supportMc2 = true;
    bool castScale = false;                  // a cast + scale form: used for calls that ask for it, and only for those
    std::function<bool(const OpDesc&, const TopoInfo&, std::string*)> opCustomCheck;
    std::function<bool(const TopoInfo&, std::string*)> topoCustomCheck;
};

struct AlgEntry {
    std::string name;             // "<Engine><Op><Strategy><Level0>[<Level1>[<Level2>]]"
    HcclCMDType op;
    HcclCommEngine engine;
    std::string executor;         // sole | sequence | parallel | concurrent | pipeline | orderpreserved
    std::vector<std::string> templates;
    AlgAttrs attrs;
    int devAlg = -1;              // DevAlg for device engines
    int hostAlg = -1;             // HostAlg for the host engine
    AlgoType family = AlgoType::MESH;   // what an HCCL_ALGO entry has to name to prefer this algorithm
    CostAgg agg = CostAgg::SUM;
    std::function<std::vector<CostCoeff>(const TopoInfo&, const OpDesc&)> costCoeff;
};

class AlgRegistry {
public:
    static AlgRegistry& Instance();
    int Register(AlgEntry e);                       // returns the index; duplicate (op,name) is rejected (-1)
    const std::vector<AlgEntry>& All() const { return algs_; }
    const AlgEntry* Find(HcclCMDType op, const std::string& name) const;
    int IndexOf(HcclCMDType op, const std::string& name) const;
    std::vector<int> ForOp(HcclCMDType op) const;
private:
    std::vector<AlgEntry> algs_;
};
struct AlgRegistrar { explicit AlgRegistrar(AlgEntry e) { AlgRegistry::Instance().Register(std::move(e)); } };
// Makes sure the translation units holding static registrations are linked in and run.
void EnsureAlgorithmsRegistered();

// "P2pAllReduceSoleMeshTwoShot" -> (engine "p2p", executor "sole", template "meshtwoshot")
// (reference algo_name_mapper.cc, hccl_tuner_plugin.h:127-134).
struct AlgNameDims { std::string engine, executor, templ; };
bool MapAlgName(const AlgEntry& e, AlgNameDims* out);

// Measured utilisation of a link class at a given per-link message size, in (0, 1].
// nRanks picks the curve measured at that GPU count (the nearest one measured; 0 = the built-in curve).
double LinkUtilisation(NetType net, double bytes, HcclCommEngine engine, int nRanks = 0);
// Replaces the link parameters and the utilisation curves with those of a measurement file (JSON, written by
// bench/sweep.py --write-link-model): {"link": {"p2pGBs": ..}, "utilisation": {"p2p": {"2": [[bytes, util], ..], "8": ..},
// "nvls": {..}}}.  Returns false and fills *err when the file cannot be read or parsed; the built-in values stay.
bool LoadLinkModelFile(const std::string& path, std::string* err);
// The file the library loads by itself on first use: HCCL_LINK_MODEL_FILE, else data/link_model.json beside the
// Python package / the library.  Empty when none exists.
std::string DefaultLinkModelPath();
// Peak figures (GB/s, us) the coefficients are built from; overridable for tests and by calibration.
struct LinkModel {
    double p2pGBs = 770.0;        // measured peer copy per direction per GPU
    double nvlsGBs = 900.0;       // nominal per-direction port rate, utilisation table carries the rest
    double nvlsReduceOutGBs = 335.0;  // reduced bytes one GPU receives per second through multimem.ld_reduce (measured, 2 and 8 GPUs)
    double nvlsStoreGBs = 515.0;      // bytes one GPU sends per second through multimem.st (measured)
    double localCopyGBs = 3200.0; // HBM read+write for a device-local copy
    double localReduceGBs = 3200.0;
    double hostMemGBs = 10.0;
    double launchUs = 2.5;        // kernel launch + first wave
    double barrierUs = 2.2;       // one cross-GPU flag round trip (8 ranks)
    double llHopUs = 1.3;         // one-way flag-in-data store visibility
    double hostStepUs = 3.0;      // one host-thread step (notify + wake)
};
LinkModel& GlobalLinkModel();

struct CostRow {
    int algIndex = -1;
    double cost = 0;        // us; <0 disabled (tuner), 0 preferred
    bool viable = false;
    bool preferred = false; // matches HCCL_ALGO
    bool tunerTouched = false;
    bool byThreshold = false; // named by the threshold tree
    std::string reason;     // why it was filtered, empty if viable
};

// Per-communicator state: cost model (which algorithms survive engine + topology filters) and tuner context.
class SelectorState {
public:
    SelectorState();
    ~SelectorState();
    bool modelReady = false;
    std::vector<int> modelAlgs[HCCL_CMD_MAX];      // surviving registry indices per op
    std::vector<std::string> modelDropReason;       // per registry index, why dropped from the model
    // tuner
    bool tunerInitTried = false;
    void* tunerHandle = nullptr;
    const HcclTunerPluginOps* tunerOps = nullptr;
    std::vector<uint8_t> tunerCtx;
    int tunerSlowCalls = 0;
    bool tieWarned[HCCL_CMD_MAX] = {false};   // the cost-tie warning is given once per operator
    bool tunerDisabled = false;
    uint64_t selections = 0;
};

struct Selection {
    int algIndex = -1;
    const AlgEntry* alg = nullptr;
    double costUs = 0;
    std::vector<CostRow> table;   // the full table, for logging and tests
};

// Builds the per-communicator model on first use, then the cost table for `op`, applies HCCL_ALGO preference and
// the tuner, and returns the cheapest viable algorithm in the best engine tier.
HcclResult SelectAlgorithm(SelectorState& st, const TopoInfo& topo, const EnvConfig& env, const OpDesc& op,
                           const std::string& commName, HcclComm commHandle, uint64_t bufferBytes, Selection* out);
// Pure helpers (unit-tested).
double EvalCost(const std::vector<CostCoeff>& segs, CostAgg agg, double bytes, HcclCommEngine engine, int nRanks = 0);
std::vector<HcclCommEngine> EngineTiers(HcclCommEngine requested);
std::string FormatCostTable(const Selection& s);
HcclResult TunerInit(SelectorState& st, const EnvConfig& env, const TopoInfo& topo, const std::string& commName,
                     HcclComm commHandle, uint64_t bufferBytes);
void TunerClose(SelectorState& st);

}  // namespace hccl
