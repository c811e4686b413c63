// Device kinds and provider names used as registration keys
// (runtime/include/brt/backends/common.h:22-30).
#pragma once
namespace brt {
namespace DeviceKind {
constexpr const char *CPU = "CPU";
constexpr const char *CUDA = "CUDA";
} // namespace DeviceKind
namespace ProviderType {
constexpr const char *BRT = "BRT";
constexpr const char *NCCL = "NCCL";
} // namespace ProviderType
} // namespace brt
