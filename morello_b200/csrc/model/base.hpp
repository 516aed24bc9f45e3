// Basic vocabulary of the scheduling model: dtypes, memory levels, shapes and the
// integer helpers the cost model is written in.
//
// Everything in this directory is HOST code of the product: it restates, for the
// Avx2 ("X86") target with default features, the parts of Morello's Spec model that
// the synthesis-database fill needs in order to enumerate candidate actions and
// their sub-Specs. Reference anchors (paths inside the Morello repository):
//   morello/src/common.rs:13-50      Dtype and its byte sizes
//   morello/src/target/cpu.rs:48-49  memory order [RF, VRF, L1, GL]
//   morello/src/target/cpu.rs:2488-2531  per-memory properties
//   morello/src/target/avx2.rs:29-65 hit costs, processors, max_mem
//   morello/src/utils.rs:123-172     bit_length / power-of-two helpers
#pragma once
#include <cstdint>
#include <cstring>
#include <string>
#include <vector>
#include <stdexcept>

namespace mrl {

using u8 = uint8_t;
using u16 = uint16_t;
using u32 = uint32_t;
using u64 = uint64_t;

// ---- dtypes (morello/src/common.rs:13-37, codes follow DtypeBimap :67-80) ----
enum Dtype : u8 { DT_U8 = 0, DT_S8 = 1, DT_U16 = 2, DT_S16 = 3, DT_U32 = 4, DT_S32 = 5, DT_F32 = 6, DT_BF16 = 7 };

inline u32 dtype_size(Dtype d) {
  switch (d) {
    case DT_U8: case DT_S8: return 1;
    case DT_U16: case DT_S16: case DT_BF16: return 2;
    default: return 4;
  }
}
inline const char* dtype_name(Dtype d) {
  static const char* n[] = {"u8", "i8", "u16", "i16", "u32", "i32", "f32", "bf16"};
  return n[d];
}

// ---- memories. The enum value is both the index into a limits vector and the
// "level" coordinate of the task grid (CpuMemoryBimap, cpu.rs:2577-2606). ----
enum Mem : u8 { RF = 0, VRF = 1, L1 = 2, GL = 3 };
constexpr int NMEM = 4;
constexpr u32 LINE_SIZE = 64;  // cpu.rs:280-282

inline bool mem_counts_registers(Mem m) { return m == RF || m == VRF; }
inline bool mem_has_layout(Mem m) { return m != RF; }
inline bool mem_is_addressed(Mem m) { return m != L1; }
inline bool mem_is_vector(Mem m) { return m == VRF; }
inline u32 mem_hit_cost(Mem m) {  // Avx2, default features (GL = 20)
  switch (m) { case L1: return 2; case GL: return 20; default: return 0; }
}
inline const char* mem_name(Mem m) {
  static const char* n[] = {"RF", "VRF", "L1", "GL"};
  return n[m];
}
// Vector register widths in bytes (cpu.rs:2508-2513).
inline const std::vector<u32>& mem_vector_bytes(Mem m) {
  static const std::vector<u32> vrf = {16, 32};
  static const std::vector<u32> none = {};
  return m == VRF ? vrf : none;
}
// cpu.rs:300-315: where a tensor living in `m` may be moved.
inline std::vector<Mem> possible_destination_memories(Mem m) {
  switch (m) {
    case RF: return {RF};
    case VRF: return {VRF};
    case L1: return {L1, RF, VRF};
    default: return {GL, L1};
  }
}
// Avx2Target::max_mem() decoded (avx2.rs:59-65).
constexpr u64 AVX2_MAX_MEM[NMEM] = {16, 16, 1024, 33554432};
constexpr u32 AVX2_PROCESSORS = 16;

// ---- integer helpers (utils.rs:123-172) ----
inline bool is_pow2(u64 n) { return n != 0 && (n & (n - 1)) == 0; }
inline u32 bit_length(u64 n) { return n == 0 ? 0 : 64 - (u32)__builtin_clzll(n); }
inline u64 bit_length_inverse(u32 c) { return c == 0 ? 0 : (u64(1) << (c - 1)); }
inline u64 next_pow2(u64 n) {  // u64::next_power_of_two (1 for 0)
  if (n <= 1) return 1;
  return u64(1) << (64 - __builtin_clzll(n - 1));
}
inline u64 next_binary_power(u64 n) { return n == 0 ? 0 : next_pow2(n); }
inline u64 prev_power_of_two(u64 n) {
  u32 hi = 63 - (u32)__builtin_clzll(n | 1);
  return (u64(1) << hi) & n;
}
inline u32 sat_add_u32(u32 a, u32 b) { u64 s = u64(a) + b; return s > 0xFFFFFFFFull ? 0xFFFFFFFFu : (u32)s; }
inline u32 sat_mul_u32(u32 a, u32 b) { u64 s = u64(a) * b; return s > 0xFFFFFFFFull ? 0xFFFFFFFFu : (u32)s; }

// ---- shapes ----
constexpr int MAX_RANK = 7;  // Conv spec shapes have rank 7; tensors have rank <= 4
struct Shape {
  u8 n = 0;
  u32 d[MAX_RANK] = {0, 0, 0, 0, 0, 0, 0};
  Shape() {}
  Shape(std::initializer_list<u32> l) { for (u32 v : l) d[n++] = v; }
  u32 operator[](int i) const { return d[i]; }
  u32& operator[](int i) { return d[i]; }
  u64 volume() const { u64 v = 1; for (int i = 0; i < n; i++) v *= d[i]; return v; }
  bool operator==(const Shape& o) const {
    if (n != o.n) return false;
    for (int i = 0; i < n; i++) if (d[i] != o.d[i]) return false;
    return true;
  }
  bool operator!=(const Shape& o) const { return !(*this == o); }
  bool all_ones() const { for (int i = 0; i < n; i++) if (d[i] != 1) return false; return true; }
  std::string str() const {
    std::string s;
    for (int i = 0; i < n; i++) { if (i) s += "x"; s += std::to_string(d[i]); }
    return s;
  }
};

// TileScale::PowerOfTwo dim_range (spec.rs:3194-3214): 1,2,4,... < dim [, dim].
inline std::vector<u32> dim_range_pow2(u32 dim, bool include_end) {
  std::vector<u32> r;
  for (u32 x = 1; x < dim; x *= 2) r.push_back(x);
  if (include_end) r.push_back(dim);
  return r;
}

struct ModelError : std::runtime_error {
  using std::runtime_error::runtime_error;
};

}  // namespace mrl
