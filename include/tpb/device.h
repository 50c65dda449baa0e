// A device is a (type, index) pair; "cpu" and "cuda" are the known types.
// Counterpart of the reference's tensorpipe/common/device.h:17-62.
#pragma once

#include <functional>
#include <string>
#include <utility>

namespace tpb {

inline const std::string kCpuDeviceType{"cpu"};
inline const std::string kCudaDeviceType{"cuda"};

struct Device {
  std::string type;
  int index = 0;

  Device() = default;
  Device(std::string t, int i) : type(std::move(t)), index(i) {}

  std::string toString() const { return type + ":" + std::to_string(index); }
  bool operator==(const Device& o) const { return type == o.type && index == o.index; }
  bool operator!=(const Device& o) const { return !(*this == o); }
  bool operator<(const Device& o) const {
    return type != o.type ? type < o.type : index < o.index;
  }
  bool isCpu() const { return type == kCpuDeviceType; }
  bool isCuda() const { return type == kCudaDeviceType; }
};

}  // namespace tpb

namespace std {
template <>
struct hash<::tpb::Device> {
  size_t operator()(const ::tpb::Device& d) const noexcept {
    return std::hash<std::string>{}(d.type) * 1000003u ^ std::hash<int>{}(d.index);
  }
};
template <>
struct hash<std::pair<::tpb::Device, ::tpb::Device>> {
  size_t operator()(const std::pair<::tpb::Device, ::tpb::Device>& p) const noexcept {
    return std::hash<::tpb::Device>{}(p.first) * 31u ^ std::hash<::tpb::Device>{}(p.second);
  }
};
}  // namespace std
