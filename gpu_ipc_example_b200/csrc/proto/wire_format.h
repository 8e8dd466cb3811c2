// Byte images of the four wire formats, as pure index arithmetic usable on the
// host (emulator, oracles) and on the device.
//
// A "transaction" is what one warp stores to a peer with one vector store: 32
// lanes x kLaneDw dwords.  Some dwords carry payload, some the 32-bit sequence
// flag of the step.  A receiver accepts a transaction only when every flag
// dword equals the expected value; because a flag sits in the same hardware
// atomic unit as the payload it guards (8 B granule for LL8/LL16, 64 B segment
// for LL128/LL512), no barrier or fence is needed around the data.
//
// Layouts (dword index inside the transaction):
//   LL8    d f d f ...                     payload k -> slot 2k, flag at 2k+1
//   LL16   d f d f | d f d f ...           payload k -> slot 2k, flag at 2k+1
//          (lane = 16 B = two self-validating 8 B granules; the reference's
//           {d0,d1,f,f} lane image needs 16 B store atomicity, which PTX does
//           not promise, so each granule carries its own flag here)
//   LL128  0..14 | F | 16..29 | p15 | F    30 payload dwords in a 128 B line
//   LL512  per 64 B segment: 15 dwords + F; the 7 dwords displaced by the first
//          seven flags are parked in slots 120..126; slot 127 is a flag.
//
// Capability parity: rt64.hpp:334-340 (8 B message), rt64.hpp:3-9 (16 B message),
// rt64_128.hpp:538-552 (120/128, flag per 64 B half, displaced word in the spare
// lane), rt64_128.hpp:3-10, 111-114, 202-226 (240/256 and 480/512 forms).
#pragma once

#include "../common/types.h"

namespace b200ipc {

template <ProtoKind K>
struct WireFormat;

template <>
struct WireFormat<ProtoKind::LL8> {
  static constexpr ProtoKind kind = ProtoKind::LL8;
  static constexpr int kLaneDw = 2;
  static constexpr int kTxnDw = 32 * kLaneDw;
  static constexpr int kPayloadDw = 32;
  static constexpr const char* name = "LL8";
  B200_HD static constexpr int payload_slot(int k) { return 2 * k; }
  B200_HD static constexpr bool is_flag_slot(int s) { return (s & 1) == 1; }
};

template <>
struct WireFormat<ProtoKind::LL16> {
  static constexpr ProtoKind kind = ProtoKind::LL16;
  static constexpr int kLaneDw = 4;
  static constexpr int kTxnDw = 32 * kLaneDw;
  static constexpr int kPayloadDw = 64;
  static constexpr const char* name = "LL16";
  B200_HD static constexpr int payload_slot(int k) { return 2 * k; }
  B200_HD static constexpr bool is_flag_slot(int s) { return (s & 1) == 1; }
};

template <>
struct WireFormat<ProtoKind::LL128> {
  static constexpr ProtoKind kind = ProtoKind::LL128;
  static constexpr int kLaneDw = 1;
  static constexpr int kTxnDw = 32;
  static constexpr int kPayloadDw = 30;
  static constexpr const char* name = "LL128";
  B200_HD static constexpr int payload_slot(int k) { return k == 15 ? 30 : k; }
  B200_HD static constexpr bool is_flag_slot(int s) { return s == 15 || s == 31; }
};

template <>
struct WireFormat<ProtoKind::LL512> {
  static constexpr ProtoKind kind = ProtoKind::LL512;
  static constexpr int kLaneDw = 4;
  static constexpr int kTxnDw = 128;
  static constexpr int kPayloadDw = 120;
  static constexpr const char* name = "LL512";
  B200_HD static constexpr int payload_slot(int k) { return (k & 15) == 15 ? 120 + (k >> 4) : k; }
  B200_HD static constexpr bool is_flag_slot(int s) { return (s & 15) == 15; }
};

template <ProtoKind K>
B200_HD constexpr int txn_bytes() { return WireFormat<K>::kTxnDw * 4; }
template <ProtoKind K>
B200_HD constexpr int payload_bytes() { return WireFormat<K>::kPayloadDw * 4; }

inline int txn_bytes_of(ProtoKind k) {
  switch (k) {
    case ProtoKind::LL8: return txn_bytes<ProtoKind::LL8>();
    case ProtoKind::LL16: return txn_bytes<ProtoKind::LL16>();
    case ProtoKind::LL128: return txn_bytes<ProtoKind::LL128>();
    default: return txn_bytes<ProtoKind::LL512>();
  }
}
inline int payload_dw_of(ProtoKind k) {
  switch (k) {
    case ProtoKind::LL8: return WireFormat<ProtoKind::LL8>::kPayloadDw;
    case ProtoKind::LL16: return WireFormat<ProtoKind::LL16>::kPayloadDw;
    case ProtoKind::LL128: return WireFormat<ProtoKind::LL128>::kPayloadDw;
    default: return WireFormat<ProtoKind::LL512>::kPayloadDw;
  }
}
inline const char* proto_name(ProtoKind k) {
  switch (k) {
    case ProtoKind::LL8: return "LL8";
    case ProtoKind::LL16: return "LL16";
    case ProtoKind::LL128: return "LL128";
    default: return "LL512";
  }
}

}  // namespace b200ipc
