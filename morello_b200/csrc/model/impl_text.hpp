// Text form of a reconstructed implementation: one line per node of the tree that results from
// re-applying, from a goal Spec down, the action the database stores for each (Spec, limits)
// (the walk of morello/src/reconstruct.rs:14-80 and FilesDatabase::get_impl,
// morello/src/db/mod.rs:505-516). The layout of a line is this library's own; the reference's
// pretty printer (morello/src/pprint.rs) prints tensors and loops of the generated code, which is
// outside the path built here.
//
//   <2 spaces per level><Spec> @ [rf, vrf, l1, gl]: #<action> <what> cost <main> peaks [..] depth <d>
#pragma once
#include "actions.hpp"

namespace mrl {

inline const char* leaf_kernel_name(u8 k) {
  static const char* n[] = {"MultAdd", "BroadcastVecMultAdd", "DotProductLoop", "Assign", "MemsetZero", "ValueZero", "VectorZero"};
  return k < 7 ? n[k] : "?";
}

inline std::string action_text(const Candidate& c) {
  switch (c.what) {
    case ACT_MOVE: {
      std::string s = "Move(operand " + std::to_string(c.arg0) + " -> " + mem_name((Mem)c.arg1);
      if (mem_has_layout((Mem)c.arg1)) s += ", layout " + c.lay.str();
      if (c.arg2) s += ", vector " + std::to_string(c.arg2);
      return s + ")";
    }
    case ACT_TILE_OUT: return "TileOut(dim " + std::to_string(c.arg0) + ", size " + std::to_string(c.arg2) + ")";
    case ACT_SPLIT: return "Split(k " + std::to_string(c.arg2) + ")";
    case ACT_KERNEL: return std::string("Kernel(") + leaf_kernel_name(c.arg0) + ")";
    default: return "ToAccum";
  }
}

inline std::string limits_text(const u64 v[NMEM]) {
  std::string s = "[";
  for (int i = 0; i < NMEM; i++) { if (i) s += ", "; s += std::to_string(v[i]); }
  return s + "]";
}

inline std::string impl_line(int level, const LogicalSpec& spec, const u64 limits[NMEM], u32 action, const std::string& what,
                             u32 main, const u64 peaks[NMEM], u32 depth) {
  return std::string((size_t)level * 2, ' ') + spec.str() + " @ " + limits_text(limits) + ": #" + std::to_string(action) + " " +
         what + " cost " + std::to_string(main) + " peaks " + limits_text(peaks) + " depth " + std::to_string(depth) + "\n";
}

}  // namespace mrl
