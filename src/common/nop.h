// A from-scratch codec for the libnop wire format that the reference speaks
// (tensorpipe/common/nop.h:55-303 glues libnop in; the format itself is libnop's).
// One prefix byte, then a payload; multi-byte values are little-endian; integers always use the
// smallest encoding that holds the value.
//
//   0x00..0x7f positive fixint      0x80..0x83 U8/U16/U32/U64     0x84..0x87 I8/I16/I32/I64
//   0x88 F32   0x89 F64             0xb8 Variant (+i32 index +value; -1 then Nil when empty)
//   0xb9 Structure (+count +members)  0xba Array (+count +elements)  0xbb Map (+count +k,v..)
//   0xbc Binary (+byte length +raw; vectors of integral types)   0xbd String (+length +bytes)
//   0xbe Nil (empty optional)       0xc0..0xff negative fixint (-64..-1)    bool = 0x00 / 0x01
//
// Structures list their members with TPB_NOP_STRUCTURE(Type, a, b, c) inside the struct; foreign
// types specialise tpb::nop::Members<Type>.
#pragma once

#include <array>
#include <cstdint>
#include <cstring>
#include <limits>
#include <map>
#include <optional>
#include <string>
#include <tuple>
#include <type_traits>
#include <unordered_map>
#include <utility>
#include <variant>
#include <vector>

namespace tpb {
namespace nop {

enum : uint8_t {
  kU8 = 0x80, kU16 = 0x81, kU32 = 0x82, kU64 = 0x83,
  kI8 = 0x84, kI16 = 0x85, kI32 = 0x86, kI64 = 0x87,
  kF32 = 0x88, kF64 = 0x89,
  kVariant = 0xb8, kStructure = 0xb9, kArray = 0xba, kMap = 0xbb,
  kBinary = 0xbc, kString = 0xbd, kNil = 0xbe,
};

class Writer {
 public:
  void byte(uint8_t b) { buf_.push_back(b); }
  void raw(const void* p, size_t n) {
    const uint8_t* c = static_cast<const uint8_t*>(p);
    buf_.insert(buf_.end(), c, c + n);
  }
  template <typename T>
  void le(T v) { raw(&v, sizeof(T)); }  // host is little-endian (x86-64 / aarch64)
  std::vector<uint8_t>& buffer() { return buf_; }
  std::vector<uint8_t> take() { return std::move(buf_); }

 private:
  std::vector<uint8_t> buf_;
};

class Reader {
 public:
  Reader(const void* p, size_t n) : p_(static_cast<const uint8_t*>(p)), end_(p_ + n) {}
  bool byte(uint8_t& b) {
    if (p_ >= end_) return false;
    b = *p_++;
    return true;
  }
  bool peek(uint8_t& b) const {
    if (p_ >= end_) return false;
    b = *p_;
    return true;
  }
  bool raw(void* out, size_t n) {
    if (static_cast<size_t>(end_ - p_) < n) return false;
    std::memcpy(out, p_, n);
    p_ += n;
    return true;
  }
  template <typename T>
  bool le(T& v) { return raw(&v, sizeof(T)); }
  size_t remaining() const { return static_cast<size_t>(end_ - p_); }

 private:
  const uint8_t* p_;
  const uint8_t* end_;
};

// ---- integers -------------------------------------------------------------------------------
inline void writeUnsigned(Writer& w, uint64_t v) {
  if (v < 0x80) w.byte(static_cast<uint8_t>(v));
  else if (v <= 0xff) { w.byte(kU8); w.le<uint8_t>(static_cast<uint8_t>(v)); }
  else if (v <= 0xffff) { w.byte(kU16); w.le<uint16_t>(static_cast<uint16_t>(v)); }
  else if (v <= 0xffffffffull) { w.byte(kU32); w.le<uint32_t>(static_cast<uint32_t>(v)); }
  else { w.byte(kU64); w.le<uint64_t>(v); }
}
inline void writeSigned(Writer& w, int64_t v) {
  if (v >= -64 && v <= 127) w.byte(static_cast<uint8_t>(static_cast<int8_t>(v)));
  else if (v >= INT8_MIN && v <= INT8_MAX) { w.byte(kI8); w.le<int8_t>(static_cast<int8_t>(v)); }
  else if (v >= INT16_MIN && v <= INT16_MAX) { w.byte(kI16); w.le<int16_t>(static_cast<int16_t>(v)); }
  else if (v >= INT32_MIN && v <= INT32_MAX) { w.byte(kI32); w.le<int32_t>(static_cast<int32_t>(v)); }
  else { w.byte(kI64); w.le<int64_t>(v); }
}
// Accepts any integer encoding whose value fits the destination (a tolerant reader).
inline bool readInteger(Reader& r, bool wantSigned, uint64_t& uout, int64_t& sout) {
  uint8_t p;
  if (!r.byte(p)) return false;
  bool neg = false;
  if (p < 0x80) { uout = p; sout = p; return true; }
  if (p >= 0xc0) { sout = static_cast<int8_t>(p); uout = static_cast<uint64_t>(sout); neg = true; return wantSigned || !neg; }
  switch (p) {
    case kU8: { uint8_t v; if (!r.le(v)) return false; uout = v; sout = v; return true; }
    case kU16: { uint16_t v; if (!r.le(v)) return false; uout = v; sout = v; return true; }
    case kU32: { uint32_t v; if (!r.le(v)) return false; uout = v; sout = v; return true; }
    case kU64: { uint64_t v; if (!r.le(v)) return false; uout = v; sout = static_cast<int64_t>(v); return true; }
    case kI8: { int8_t v; if (!r.le(v)) return false; sout = v; uout = static_cast<uint64_t>(sout); return wantSigned || v >= 0; }
    case kI16: { int16_t v; if (!r.le(v)) return false; sout = v; uout = static_cast<uint64_t>(sout); return wantSigned || v >= 0; }
    case kI32: { int32_t v; if (!r.le(v)) return false; sout = v; uout = static_cast<uint64_t>(sout); return wantSigned || v >= 0; }
    case kI64: { int64_t v; if (!r.le(v)) return false; sout = v; uout = static_cast<uint64_t>(sout); return wantSigned || v >= 0; }
    default: return false;
  }
}
inline bool readSize(Reader& r, uint64_t& n) {
  int64_t s;
  return readInteger(r, false, n, s);
}

// ---- generic encode/decode ------------------------------------------------------------------
template <typename T, typename Enable = void>
struct Codec;  // Codec<T>::write(Writer&, const T&), ::read(Reader&, T&) -> bool

template <typename T>
void write(Writer& w, const T& v) { Codec<T>::write(w, v); }
template <typename T>
bool read(Reader& r, T& v) { return Codec<T>::read(r, v); }

template <>
struct Codec<bool> {
  static void write(Writer& w, const bool& v) { w.byte(v ? 1 : 0); }
  static bool read(Reader& r, bool& v) {
    uint8_t b;
    if (!r.byte(b) || b > 1) return false;
    v = b != 0;
    return true;
  }
};

template <typename T>
struct Codec<T, std::enable_if_t<std::is_integral_v<T> && !std::is_same_v<T, bool>>> {
  static void write(Writer& w, const T& v) {
    if constexpr (std::is_signed_v<T>) writeSigned(w, static_cast<int64_t>(v));
    else writeUnsigned(w, static_cast<uint64_t>(v));
  }
  static bool read(Reader& r, T& v) {
    uint64_t u; int64_t s;
    if (!readInteger(r, std::is_signed_v<T>, u, s)) return false;
    if constexpr (std::is_signed_v<T>) {
      if (s < static_cast<int64_t>(std::numeric_limits<T>::min()) ||
          s > static_cast<int64_t>(std::numeric_limits<T>::max())) return false;
      v = static_cast<T>(s);
    } else {
      if (u > static_cast<uint64_t>(std::numeric_limits<T>::max())) return false;
      v = static_cast<T>(u);
    }
    return true;
  }
};

template <typename T>
struct Codec<T, std::enable_if_t<std::is_enum_v<T>>> {
  using U = std::underlying_type_t<T>;
  static void write(Writer& w, const T& v) { Codec<U>::write(w, static_cast<U>(v)); }
  static bool read(Reader& r, T& v) {
    U u;
    if (!Codec<U>::read(r, u)) return false;
    v = static_cast<T>(u);
    return true;
  }
};

template <>
struct Codec<float> {
  static void write(Writer& w, const float& v) { w.byte(kF32); w.le(v); }
  static bool read(Reader& r, float& v) { uint8_t p; return r.byte(p) && p == kF32 && r.le(v); }
};
template <>
struct Codec<double> {
  static void write(Writer& w, const double& v) { w.byte(kF64); w.le(v); }
  static bool read(Reader& r, double& v) { uint8_t p; return r.byte(p) && p == kF64 && r.le(v); }
};

template <>
struct Codec<std::string> {
  static void write(Writer& w, const std::string& v) {
    w.byte(kString);
    writeUnsigned(w, v.size());
    w.raw(v.data(), v.size());
  }
  static bool read(Reader& r, std::string& v) {
    uint8_t p; uint64_t n;
    if (!r.byte(p) || p != kString || !readSize(r, n) || n > r.remaining()) return false;
    v.resize(n);
    return r.raw(v.data(), n);
  }
};

template <typename T>
struct Codec<std::vector<T>> {
  static constexpr bool kBinaryForm = std::is_integral_v<T> && !std::is_same_v<T, bool>;
  static void write(Writer& w, const std::vector<T>& v) {
    if constexpr (kBinaryForm) {
      w.byte(kBinary);
      writeUnsigned(w, v.size() * sizeof(T));
      w.raw(v.data(), v.size() * sizeof(T));
    } else {
      w.byte(kArray);
      writeUnsigned(w, v.size());
      for (const auto& e : v) nop::write(w, e);
    }
  }
  static bool read(Reader& r, std::vector<T>& v) {
    uint8_t p; uint64_t n;
    if (!r.byte(p)) return false;
    if constexpr (kBinaryForm) {
      if (p != kBinary || !readSize(r, n) || n > r.remaining() || n % sizeof(T) != 0) return false;
      v.resize(n / sizeof(T));
      return r.raw(v.data(), n);
    } else {
      if (p != kArray || !readSize(r, n) || n > r.remaining()) return false;
      v.clear();
      v.resize(n);
      for (auto& e : v) if (!nop::read(r, e)) return false;
      return true;
    }
  }
};

template <typename T, size_t N>
struct Codec<std::array<T, N>> {
  static_assert(std::is_integral_v<T>, "only integral std::array is encoded (as Binary)");
  static void write(Writer& w, const std::array<T, N>& v) {
    w.byte(kBinary);
    writeUnsigned(w, N * sizeof(T));
    w.raw(v.data(), N * sizeof(T));
  }
  static bool read(Reader& r, std::array<T, N>& v) {
    uint8_t p; uint64_t n;
    if (!r.byte(p) || p != kBinary || !readSize(r, n) || n != N * sizeof(T)) return false;
    return r.raw(v.data(), n);
  }
};

template <typename A, typename B>
struct Codec<std::pair<A, B>> {
  static void write(Writer& w, const std::pair<A, B>& v) {
    w.byte(kArray);
    writeUnsigned(w, 2);
    nop::write(w, v.first);
    nop::write(w, v.second);
  }
  static bool read(Reader& r, std::pair<A, B>& v) {
    uint8_t p; uint64_t n;
    if (!r.byte(p) || p != kArray || !readSize(r, n) || n != 2) return false;
    return nop::read(r, v.first) && nop::read(r, v.second);
  }
};

template <typename M>
struct MapCodec {
  static void write(Writer& w, const M& m) {
    w.byte(kMap);
    writeUnsigned(w, m.size());
    for (const auto& kv : m) {
      nop::write(w, kv.first);
      nop::write(w, kv.second);
    }
  }
  static bool read(Reader& r, M& m) {
    uint8_t p; uint64_t n;
    if (!r.byte(p) || p != kMap || !readSize(r, n) || n > r.remaining()) return false;
    m.clear();
    for (uint64_t i = 0; i < n; ++i) {
      typename M::key_type k;
      typename M::mapped_type v;
      if (!nop::read(r, k) || !nop::read(r, v)) return false;
      m.emplace(std::move(k), std::move(v));
    }
    return true;
  }
};
template <typename K, typename V, typename H, typename E, typename A>
struct Codec<std::unordered_map<K, V, H, E, A>> : MapCodec<std::unordered_map<K, V, H, E, A>> {};
template <typename K, typename V, typename C, typename A>
struct Codec<std::map<K, V, C, A>> : MapCodec<std::map<K, V, C, A>> {};

// optional<T>: Nil when empty, otherwise exactly T's encoding (no extra prefix).
template <typename T>
struct Codec<std::optional<T>> {
  static void write(Writer& w, const std::optional<T>& v) {
    if (v) nop::write(w, *v);
    else w.byte(kNil);
  }
  static bool read(Reader& r, std::optional<T>& v) {
    uint8_t p;
    if (!r.peek(p)) return false;
    if (p == kNil) {
      r.byte(p);
      v.reset();
      return true;
    }
    T tmp;
    if (!nop::read(r, tmp)) return false;
    v = std::move(tmp);
    return true;
  }
};

// variant<Ts...>: prefix, active index as a signed integer, then the value.
// std::monostate as first alternative is not used; an "empty" variant is index -1 + Nil.
template <typename... Ts>
struct Codec<std::variant<Ts...>> {
  using V = std::variant<Ts...>;
  static void write(Writer& w, const V& v) {
    w.byte(kVariant);
    if (v.valueless_by_exception()) {
      writeSigned(w, -1);
      w.byte(kNil);
      return;
    }
    writeSigned(w, static_cast<int32_t>(v.index()));
    std::visit([&](const auto& x) { nop::write(w, x); }, v);
  }
  template <size_t I = 0>
  static bool readAlt(Reader& r, V& v, size_t idx) {
    if constexpr (I >= sizeof...(Ts)) {
      return false;
    } else {
      if (idx == I) {
        std::variant_alternative_t<I, V> x;
        if (!nop::read(r, x)) return false;
        v.template emplace<I>(std::move(x));
        return true;
      }
      return readAlt<I + 1>(r, v, idx);
    }
  }
  static bool read(Reader& r, V& v) {
    uint8_t p;
    if (!r.byte(p) || p != kVariant) return false;
    int32_t idx;
    if (!nop::read(r, idx) || idx < 0) return false;
    return readAlt(r, v, static_cast<size_t>(idx));
  }
};

// ---- structures -----------------------------------------------------------------------------
template <typename T, typename = void>
struct Members;  // Members<T>::tie(T&) -> std::tuple<member&...>

template <typename T>
struct HasMembers {
  template <typename U> static auto test(int) -> decltype(Members<U>::tie(std::declval<U&>()), std::true_type{});
  template <typename> static std::false_type test(...);
  static constexpr bool value = decltype(test<T>(0))::value;
};

template <typename T>
struct Codec<T, std::enable_if_t<HasMembers<T>::value>> {
  static void write(Writer& w, const T& v) {
    auto t = Members<T>::tie(const_cast<T&>(v));
    w.byte(kStructure);
    writeUnsigned(w, std::tuple_size_v<decltype(t)>);
    std::apply([&](auto&... m) { (nop::write(w, m), ...); }, t);
  }
  static bool read(Reader& r, T& v) {
    uint8_t p; uint64_t n;
    auto t = Members<T>::tie(v);
    if (!r.byte(p) || p != kStructure || !readSize(r, n) || n != std::tuple_size_v<decltype(t)>) return false;
    return std::apply([&](auto&... m) { return (nop::read(r, m) && ...); }, t);
  }
};

template <typename T>
struct Members<T, std::void_t<decltype(std::declval<T&>().tpbNopTie())>> {
  static auto tie(T& v) { return v.tpbNopTie(); }
};

#define TPB_NOP_STRUCTURE(Type, ...) \
  auto tpbNopTie() { return std::tie(__VA_ARGS__); }

// Foreign types: specialise Members<Type> at tpb::nop scope:
//   template <> struct Members<Foo, void> { static auto tie(Foo& v) { return std::tie(v.a, v.b); } };

// ---- convenience ----------------------------------------------------------------------------
template <typename T>
std::vector<uint8_t> encode(const T& v) {
  Writer w;
  write(w, v);
  return w.take();
}
template <typename T>
bool decode(const void* p, size_t n, T& v) {
  Reader r(p, n);
  return read(r, v) && r.remaining() == 0;
}

}  // namespace nop
}  // namespace tpb
