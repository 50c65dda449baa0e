// Control messages the core exchanges, in the exact member order a reference peer expects
// (tensorpipe/core/nop_types.h:26-80): Packet = Variant<SpontaneousConnection,
// RequestedConnection>, Brochure, BrochureAnswer, Descriptor, DescriptorReply.
#pragma once

#include <string>
#include <unordered_map>
#include <variant>
#include <vector>

#include <tpb/device.h>
#include <tpb/message.h>

#include "common/nop.h"

namespace tpb {

struct SpontaneousConnection {
  std::string contextName;
  TPB_NOP_STRUCTURE(SpontaneousConnection, contextName)
};

struct RequestedConnection {
  uint64_t registrationId = 0;
  TPB_NOP_STRUCTURE(RequestedConnection, registrationId)
};

using Packet = std::variant<SpontaneousConnection, RequestedConnection>;

struct Brochure {
  std::unordered_map<std::string, std::string> transportDomainDescriptors;
  std::unordered_map<std::string, std::unordered_map<Device, std::string>> channelDeviceDescriptors;
  TPB_NOP_STRUCTURE(Brochure, transportDomainDescriptors, channelDeviceDescriptors)
};

struct BrochureAnswer {
  std::string transport;
  std::string address;
  std::unordered_map<uint64_t, uint64_t> transportRegistrationIds;
  std::string transportDomainDescriptor;
  std::unordered_map<std::string, std::vector<uint64_t>> channelRegistrationIds;
  std::unordered_map<std::string, std::unordered_map<Device, std::string>> channelDeviceDescriptors;
  std::unordered_map<std::pair<Device, Device>, std::string> channelForDevicePair;
  TPB_NOP_STRUCTURE(
      BrochureAnswer, transport, address, transportRegistrationIds, transportDomainDescriptor,
      channelRegistrationIds, channelDeviceDescriptors, channelForDevicePair)
};

struct DescriptorReply {
  std::vector<Device> targetDevices;
  TPB_NOP_STRUCTURE(DescriptorReply, targetDevices)
};

namespace nop {
template <>
struct Members<Device, void> {
  static auto tie(Device& v) { return std::tie(v.type, v.index); }
};
template <>
struct Members<Descriptor::Payload, void> {
  static auto tie(Descriptor::Payload& v) { return std::tie(v.length, v.metadata); }
};
template <>
struct Members<Descriptor::Tensor, void> {
  static auto tie(Descriptor::Tensor& v) {
    return std::tie(v.length, v.sourceDevice, v.targetDevice, v.metadata);
  }
};
template <>
struct Members<Descriptor, void> {
  static auto tie(Descriptor& v) { return std::tie(v.metadata, v.payloads, v.tensors); }
};
}  // namespace nop

}  // namespace tpb
