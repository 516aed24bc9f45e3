// TEST INFRASTRUCTURE — NOT PART OF THE PRODUCT PATH. Command-line front end of the
// CPU oracle: `oracle_cli precompute <size> [threads] [through] [dtype_mask] [budget_s] [cache]`
// mirrors `precompute --target avx2 --through <..> <size>` (precompute/src/main.rs:59-90)
// and `oracle_cli matmul <size> [dtype]` mirrors `morello matmul <size>`
// (frontend/src/main.rs:192-204,287-296).
#include "oracle.hpp"
#include <cstdio>
#include <cstdlib>
#include <cstring>
using namespace orc;

static LogicalSpec matmul_goal(u32 size, Dtype dt) {
  LogicalSpec l;
  l.kind = K_MATMUL;
  l.dtype = dt;
  l.serial_only = true;
  l.spec_shape = Shape{1, size, size, size};
  for (int i = 0; i < 3; i++) {
    l.aux[i].mem = GL;
    l.aux[i].layout = layout_row_major(l.operand_shape(i));
  }
  return l;
}

int main(int argc, char** argv) {
  if (argc < 3) {
    fprintf(stderr, "usage: %s precompute <size> [threads] [through 0|1|2] [dtype_mask] [budget_s] | matmul <size> [u32|f32]\n", argv[0]);
    return 2;
  }
  try {
    Database db;
    if (!strcmp(argv[1], "precompute")) {
      u32 size = atoi(argv[2]);
      int threads = argc > 3 ? atoi(argv[3]) : 1;
      int through = argc > 4 ? atoi(argv[4]) : 2;
      int mask = argc > 5 ? atoi(argv[5]) : 3;
      double budget = argc > 6 ? atof(argv[6]) : 0;
      bool cache = argc > 7 ? atoi(argv[7]) != 0 : false;
      std::vector<Dtype> dts;
      if (mask & 1) dts.push_back(DT_U32);
      if (mask & 2) dts.push_back(DT_F32);
      bool fin = false;
      PrecomputeReport r = precompute(db, size, (Through)through, dts, threads, budget, &fin, cache);
      printf("{\"size\": %u, \"threads\": %d, \"seconds\": %.3f, \"puts\": %llu, \"logical_specs\": %llu, \"solves\": %llu, "
             "\"finished\": %s, \"dominance_conflicts\": %llu, \"puts_per_s\": %.1f}\n",
             size, threads, r.seconds, (unsigned long long)r.puts, (unsigned long long)r.logical_specs,
             (unsigned long long)r.solves, fin ? "true" : "false", (unsigned long long)db.dominance_conflicts.load(),
             r.puts / r.seconds);
    } else {
      u32 size = atoi(argv[2]);
      Dtype dt = (argc > 3 && !strcmp(argv[3], "f32")) ? DT_F32 : DT_U32;
      LogicalSpec goal = matmul_goal(size, dt);
      Limits top = {AVX2_MAX_MEM[0], AVX2_MAX_MEM[1], AVX2_MAX_MEM[2], AVX2_MAX_MEM[3]};
      Search s(db);
      Decision d = s.solve(goal, top);
      printf("%s -> found=%d action=%u main=%u peaks=[%llu,%llu,%llu,%llu] depth=%u puts=%llu solves=%llu conflicts=%llu\n",
             goal.str().c_str(), d.found, d.action, d.cost.main, (unsigned long long)d.cost.peaks[0],
             (unsigned long long)d.cost.peaks[1], (unsigned long long)d.cost.peaks[2], (unsigned long long)d.cost.peaks[3],
             d.cost.depth, (unsigned long long)db.puts.load(), (unsigned long long)s.stats.solves,
             (unsigned long long)db.dominance_conflicts.load());
    }
  } catch (const std::exception& e) {
    fprintf(stderr, "error: %s\n", e.what());
    return 1;
  }
  return 0;
}
