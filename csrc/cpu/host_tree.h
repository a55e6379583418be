// Algorithm trees for the tree-interpreting executor.
//
// The reference's experimental recursive executor describes an algorithm as a
// tree (AlgoExecDesc: SEQUENCE / PARALLEL / OMNIPIPE nodes with template
// leaves, experimental/ops/op_common/recursive_executor/*, design in
// docs/en/rfcs/0003-executor-template-refactor.md) and runs every combination
// through one executor instead of one hand-written executor per combination.
// Here the tree comes as text in HCCL_ALGO_TREE:
//
//   node := leaf | seq(node, node[, node]) | par(node, node[, shareA:shareB]) | rev(node)
//   leaf := mesh | ring | nhr | rhd | nb
//
//   leaf          the template runs on every level it is given, taken as one flat group
//   seq(a, b, c)  child i owns topology level i: ReduceScatter with a on level 0,
//                 the rest of the tree on the slice that is left, AllGather with a
//                 on the way back; the last child takes all remaining levels
//   par(a, b)     the data is split in two parts in proportion shareA : shareB
//                 (default: the mesh : CLOS bandwidth shares) and the children run
//                 on separate queues
//   rev(a)        a sees the levels in reverse order (inter-server first), which is
//                 how the Parallel executor runs its second half
#pragma once
#include <memory>
#include <string>
#include <vector>

namespace hccl {

struct AlgoTreeNode {
    enum class Kind { LEAF, SEQ, PAR, REV } kind = Kind::LEAF;
    std::string leaf;                                   // lower-case template name
    std::vector<std::unique_ptr<AlgoTreeNode>> kids;
    double shareA = 0, shareB = 0;                      // PAR: 0,0 = default shares
};

bool ParseAlgoTree(const std::string& text, std::unique_ptr<AlgoTreeNode>* out, std::string* err);
std::string AlgoTreeText(const AlgoTreeNode& n);        // canonical text of a tree
uint32_t AlgoTreeQueues(const AlgoTreeNode& n);         // execution queues the tree uses
uint32_t AlgoTreeMinLevels(const AlgoTreeNode& n);      // topology levels the tree needs

}  // namespace hccl
