#include <mutex>
#include "selector.h"

namespace hccl {
void RegisterDeviceAlgorithms();
void RegisterHostAlgorithms();

void EnsureAlgorithmsRegistered()
{
    static std::once_flag once;
    std::call_once(once, [] {
        RegisterDeviceAlgorithms();
        RegisterHostAlgorithms();
    });
}
}  // namespace hccl
