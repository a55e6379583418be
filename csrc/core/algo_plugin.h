// Host of the algorithm plugin (HCCL_ALGO_PLUGIN_PATH): loads the table once per process and offers every operator
// call to it before the built-in selector runs.
#pragma once
#include <string>
#include "hccl/hccl_algo_plugin.h"

namespace hccl {
class CommImpl;
struct OpParam;
// Returns true when the plugin claimed and executed the call; *result then holds its return code and *algName its name.
bool AlgoPluginTryExecute(CommImpl* comm, const OpParam& p, HcclResult* result, std::string* algName);
HcclResult AlgoPluginQueryAlgs(const char* opName, char* buf, uint32_t bufLen, uint32_t* count);
void AlgoPluginReload();   // drop the loaded plugin so that the next call re-reads HCCL_ALGO_PLUGIN_PATH (tests)
}  // namespace hccl
