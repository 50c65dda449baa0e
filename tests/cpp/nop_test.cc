// Golden-byte tests of the control-message codec: the bytes below are what a libnop writer
// emits for these values (prefix byte, smallest integer encoding, little-endian), so a
// reference peer can parse our frames and we can parse theirs.
#include "common/nop.h"
#include "core/nop_types.h"
#include "test_util.h"

using namespace tpb;

namespace {
std::string hex(const std::vector<uint8_t>& v) {
  static const char* d = "0123456789abcdef";
  std::string s;
  for (uint8_t b : v) {
    s.push_back(d[b >> 4]);
    s.push_back(d[b & 15]);
  }
  return s;
}
template <typename T>
void roundTrip(const T& v, const std::string& golden) {
  auto bytes = nop::encode(v);
  EXPECT_EQ(hex(bytes), golden);
  T back{};
  EXPECT_TRUE(nop::decode(bytes.data(), bytes.size(), back));
  EXPECT_EQ(hex(nop::encode(back)), golden);
}
}  // namespace

TPB_TEST(Nop, Integers) {
  roundTrip<uint64_t>(5, "05");
  roundTrip<uint64_t>(127, "7f");
  roundTrip<uint64_t>(128, "8080");
  roundTrip<uint64_t>(300, "812c01");
  roundTrip<uint64_t>(70000, "8270110100");
  roundTrip<uint64_t>(1ull << 40, "830000000000010000");
  roundTrip<int>(0, "00");
  roundTrip<int>(-1, "ff");
  roundTrip<int>(-64, "c0");
  roundTrip<int>(-65, "84bf");
  roundTrip<int>(200, "85c800");
  roundTrip<int>(-40000, "86c063ffff");
  roundTrip<int64_t>(-(1ll << 40), "870000000000ffffff");
  roundTrip<bool>(true, "01");
  roundTrip<bool>(false, "00");
}

TPB_TEST(Nop, StringsAndContainers) {
  roundTrip<std::string>("", "bd00");
  roundTrip<std::string>("uv", "bd027576");
  roundTrip<std::vector<uint64_t>>({1, 2}, "bc1001000000000000000200000000000000");
  roundTrip<std::vector<std::string>>({"a", "bc"}, "ba02bd0161bd026263");
  roundTrip<std::pair<int, std::string>>({3, "x"}, "ba0203bd0178");
  roundTrip<std::map<std::string, uint64_t>>({{"k", 9}}, "bb01bd016b09");
  roundTrip<std::optional<std::string>>(std::nullopt, "be");
  roundTrip<std::optional<std::string>>(std::string("z"), "bd017a");
  roundTrip<float>(1.0f, "880000803f");
}

TPB_TEST(Nop, CoreStructures) {
  roundTrip<Device>(Device("cuda", 3), "b902bd046375646103");
  Packet hello = SpontaneousConnection{"ctx"};
  roundTrip<Packet>(hello, "b800b901bd03637478");
  Packet req = RequestedConnection{258};
  roundTrip<Packet>(req, "b801b901810201");

  Descriptor d;
  d.metadata = "m";
  d.payloads.push_back({4, "p"});
  Descriptor::Tensor t;
  t.length = 1024;
  t.sourceDevice = Device("cpu", 0);
  t.metadata = "";
  d.tensors.push_back(t);
  roundTrip<Descriptor>(d,
                        "b903bd016d"            // metadata
                        "ba01b90204bd0170"      // payloads [(4,"p")]
                        "ba01b904810004"        // tensors [ (1024,
                        "b902bd0363707500"      //   Device(cpu,0),
                        "be"                    //   no target device,
                        "bd00");                //   "")]
  DescriptorReply r;
  r.targetDevices.push_back(Device("cuda", 0));
  roundTrip<DescriptorReply>(r, "b901ba01b902bd046375646100");
}

TPB_TEST(Nop, BrochureRoundTrip) {
  Brochure b;
  b.transportDomainDescriptors["uv"] = "uv:*";
  b.channelDeviceDescriptors["basic"][Device("cpu", 0)] = "any";
  auto bytes = nop::encode(b);
  EXPECT_EQ(hex(bytes), "b902bb01bd027576bd0475763a2abb01bd056261736963bb01b902bd0363707500bd03616e79");
  Brochure back;
  EXPECT_TRUE(nop::decode(bytes.data(), bytes.size(), back));
  EXPECT_EQ(back.channelDeviceDescriptors["basic"][Device("cpu", 0)], std::string("any"));

  BrochureAnswer a;
  a.transport = "uv";
  a.address = "127.0.0.1:1";
  a.transportRegistrationIds[1] = 7;
  a.channelRegistrationIds["basic"] = {3};
  a.channelForDevicePair[{Device("cpu", 0), Device("cpu", 0)}] = "basic";
  auto ab = nop::encode(a);
  BrochureAnswer a2;
  EXPECT_TRUE(nop::decode(ab.data(), ab.size(), a2));
  EXPECT_EQ(a2.channelRegistrationIds["basic"].size(), size_t(1));
  EXPECT_EQ(a2.transportRegistrationIds[1], uint64_t(7));
  auto key = std::make_pair(Device("cpu", 0), Device("cpu", 0));
  EXPECT_EQ(a2.channelForDevicePair[key], std::string("basic"));
}

TPB_TEST(Nop, RejectsMalformed) {
  std::string s;
  uint8_t truncated[] = {0xbd, 0x05, 'a'};
  EXPECT_FALSE(nop::decode(truncated, sizeof(truncated), s));
  uint8_t wrongPrefix[] = {0xbc, 0x01, 'a'};
  EXPECT_FALSE(nop::decode(wrongPrefix, sizeof(wrongPrefix), s));
  uint8_t trailing[] = {0xbd, 0x01, 'a', 0x00};
  EXPECT_FALSE(nop::decode(trailing, sizeof(trailing), s));
  uint32_t small;
  uint8_t big[] = {0x83, 0, 0, 0, 0, 1, 0, 0, 0};
  EXPECT_FALSE(nop::decode(big, sizeof(big), small));
}

// Whatever arrives on the wire, decoding either succeeds or says no: it never crashes, never loops
// and never allocates more than the input could justify. Valid encodings of every core structure
// are mutated (bit flips, truncations, spliced garbage) and random bytes are thrown in as well.
#include <random>

TPB_TEST(Nop, DecodersSurviveMutatedAndRandomInput) {
  std::vector<std::vector<uint8_t>> seeds;
  {
    Packet hello = SpontaneousConnection{"some-context"};
    seeds.push_back(nop::encode(hello));
    Packet req = RequestedConnection{123456789};
    seeds.push_back(nop::encode(req));
    Brochure b;
    b.transportDomainDescriptors["uv"] = "uv:*";
    b.transportDomainDescriptors["shm"] = "tpbshm1:abc";
    b.channelDeviceDescriptors["basic"][Device("cpu", 0)] = "any";
    b.channelDeviceDescriptors["cuda_p2p"][Device("cuda", 1)] = "GPU-xyz";
    seeds.push_back(nop::encode(b));
    BrochureAnswer a;
    a.transport = "uv";
    a.address = "127.0.0.1:1";
    a.transportRegistrationIds[1] = 7;
    a.channelRegistrationIds["basic"] = {3, 4, 5};
    a.channelForDevicePair[{Device("cpu", 0), Device("cuda", 2)}] = "cuda_basic";
    seeds.push_back(nop::encode(a));
    Descriptor d;
    d.metadata = std::string(40, 'm');
    d.payloads.push_back({4, "p"});
    d.payloads.push_back({1u << 20, ""});
    for (int i = 0; i < 5; ++i) {
      Descriptor::Tensor t;
      t.length = 1024u * (i + 1);
      t.sourceDevice = Device(i % 2 ? "cuda" : "cpu", i);
      if (i % 2) t.targetDevice = Device("cuda", 7 - i);
      t.metadata = std::string(i, 't');
      d.tensors.push_back(t);
    }
    seeds.push_back(nop::encode(d));
    DescriptorReply r;
    r.targetDevices.push_back(Device("cuda", 0));
    r.targetDevices.push_back(Device("cpu", 0));
    seeds.push_back(nop::encode(r));
  }
  std::mt19937 rng(20240607);
  size_t accepted = 0, rejected = 0;
  auto tryAll = [&](const std::vector<uint8_t>& bytes) {
    Packet p;
    Brochure b;
    BrochureAnswer a;
    Descriptor d;
    DescriptorReply r;
    std::string s;
    std::vector<uint64_t> v;
    bool any = nop::decode(bytes.data(), bytes.size(), p);
    any |= nop::decode(bytes.data(), bytes.size(), b);
    any |= nop::decode(bytes.data(), bytes.size(), a);
    any |= nop::decode(bytes.data(), bytes.size(), d);
    any |= nop::decode(bytes.data(), bytes.size(), r);
    any |= nop::decode(bytes.data(), bytes.size(), s);
    any |= nop::decode(bytes.data(), bytes.size(), v);
    (any ? accepted : rejected)++;
    // A decoded descriptor never claims more entries than the input has bytes.
    EXPECT_TRUE(d.tensors.size() <= bytes.size() && d.payloads.size() <= bytes.size());
  };
  for (int iter = 0; iter < 20000; ++iter) {
    std::vector<uint8_t> bytes = seeds[rng() % seeds.size()];
    switch (rng() % 5) {
      case 0:  // flip a few bits
        for (int k = 0, n = 1 + rng() % 4; k < n && !bytes.empty(); ++k) bytes[rng() % bytes.size()] ^= 1u << (rng() % 8);
        break;
      case 1:  // truncate
        bytes.resize(rng() % (bytes.size() + 1));
        break;
      case 2:  // overwrite a run with garbage (length fields become huge)
        for (size_t k = rng() % bytes.size(), n = 0; k < bytes.size() && n < 9; ++k, ++n) bytes[k] = static_cast<uint8_t>(rng());
        break;
      case 3:  // splice two encodings
        bytes.resize(rng() % (bytes.size() + 1));
        {
          const auto& other = seeds[rng() % seeds.size()];
          bytes.insert(bytes.end(), other.begin() + rng() % other.size(), other.end());
        }
        break;
      default:  // pure noise
        bytes.resize(rng() % 64);
        for (auto& x : bytes) x = static_cast<uint8_t>(rng());
    }
    tryAll(bytes);
  }
  for (const auto& s : seeds) tryAll(s);
  EXPECT_TRUE(accepted >= seeds.size());  // the untouched encodings, at the very least
  EXPECT_TRUE(rejected > 10000);          // and most mutations are refused
}
