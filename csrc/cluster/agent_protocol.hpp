// Wire protocol between the cluster manager (head) and the per-node agents.
//
// Parity: the reference frames every request and reply with an 8-byte header
// {u16 command, u16 status, u32 payload length} and defines PING, REGISTER,
// DEREGISTER, SHADER_LOAD, SHADER_RUN, SHADER_SYNC, STATS and SHUTDOWN
// (csrc/agent/Protocol.hpp:14-84).  The same framing is used here; the shader
// commands become KERNEL_LOAD / KERNEL_RUN / KERNEL_SYNC and keep their
// numeric values.
#pragma once

#include <cstdint>
#include <string>
#include <vector>

namespace mccl {

enum class AgentCmd : uint16_t {
  PING = 1,
  REGISTER = 2,      // payload: u32 region id, u64 length
  DEREGISTER = 3,    // payload: u32 region id
  KERNEL_LOAD = 4,   // payload: kernel name
  KERNEL_RUN = 5,    // payload: u16 name length, name, u64 offset, u64 count
  KERNEL_SYNC = 6,
  STATS = 7,         // reply payload: "key=value\n" lines
  SHUTDOWN = 8,
};

enum class AgentStatus : uint16_t { OK = 0, ERROR = 1, UNKNOWN_COMMAND = 2, NOT_FOUND = 3 };

#pragma pack(push, 1)
struct AgentHeader {
  uint16_t cmd;
  uint16_t status;
  uint32_t payload_len;
};
#pragma pack(pop)
static_assert(sizeof(AgentHeader) == 8, "agent header is 8 bytes on the wire");

constexpr uint32_t kAgentMaxPayload = 1u << 20;

inline void put_u16(std::vector<uint8_t>& b, uint16_t v) { b.push_back(v & 0xff); b.push_back(v >> 8); }
inline void put_u32(std::vector<uint8_t>& b, uint32_t v) { for (int i = 0; i < 4; ++i) b.push_back((v >> (8 * i)) & 0xff); }
inline void put_u64(std::vector<uint8_t>& b, uint64_t v) { for (int i = 0; i < 8; ++i) b.push_back((v >> (8 * i)) & 0xff); }
inline uint16_t get_u16(const uint8_t* p) { return static_cast<uint16_t>(p[0] | (p[1] << 8)); }
inline uint32_t get_u32(const uint8_t* p) { uint32_t v = 0; for (int i = 0; i < 4; ++i) v |= static_cast<uint32_t>(p[i]) << (8 * i); return v; }
inline uint64_t get_u64(const uint8_t* p) { uint64_t v = 0; for (int i = 0; i < 8; ++i) v |= static_cast<uint64_t>(p[i]) << (8 * i); return v; }

}  // namespace mccl
