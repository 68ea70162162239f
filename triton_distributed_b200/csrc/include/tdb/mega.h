// Host API of the decode megakernel: task / op records, the C++ task-graph scheduler and the launcher.
#pragma once
#include <stdint.h>

#include <string>
#include <vector>

#include "api.h"

namespace tdb {

enum MegaTaskType : int32_t {
  kTaskRmsNorm = 1,      // a0 = row
  kTaskLinear = 2,       // a0 = 128-column tile, a1 = K split
  kTaskRopeKv = 3,       // a0 = token
  kTaskAttnSplit = 4,    // a0 = sequence, a1 = KV split, a2 = kv head * head chunks + chunk
  kTaskAttnCombine = 5,  // a0 = sequence
  kTaskSiluMul = 6,      // a0 = row
  kTaskPrefetch = 7,     // a0 = chunk of the byte range that is requested into L2 (cp.async.bulk.prefetch.L2)
  kTaskBarrier = 8,      // one task: barrier over all ranks (epoch flags in the heap)
  kTaskAllReduce = 9,    // a0 = column chunk of a stand-alone all-reduce of a [batch, N] bf16 tensor
};

struct MegaTask {
  int32_t type;
  int32_t dep_idx, dep_need;   // scoreboard slot that must have reached dep_need (-1: none)
  int32_t out_idx;             // scoreboard slot bumped when the task (linear: the output tile) is complete
  int32_t op;
  int32_t a0, a1, a2, a3;
  int32_t pad[7];
};
static_assert(sizeof(MegaTask) == 64, "MegaTask is 64 bytes");

// Operator record; the meaning of p / i / f depends on the task type (see megakernel.cu).
struct MegaOp {
  void* p[8];
  int32_t i[12];
  float f[4];
};

struct MegaLaunchArgs {
  const MegaTask* tasks;          // device, sorted by SM
  const int32_t* queue_offsets;   // device [grid + 1]
  const MegaOp* ops;              // device
  const void* tmaps;              // device array of 128-byte tensor maps (64-byte aligned)
  int32_t* scoreboard;            // device [scoreboard_size]
  int scoreboard_size;
  float* acc;
  uint32_t* counters;
  CtxDev* ctx;
  SymmInfoHost symm;
  int batch;
  int grid;
  int use_multimem;
  void* profile_buf;              // uint64 buffer or null
};
cudaError_t launch_megakernel(const MegaLaunchArgs& a, cudaStream_t stream);
int megakernel_mpad(int batch);

// Task graph -> per-SM queues.  Stages are appended in topological order; a stage depends on at most one earlier
// stage (all of its completion units).  Matches the reference's Graph / enque_tasks / work-queue tensors
// (mega_triton_kernel/core/graph.py:101-157, scheduler.py:41-168).
class MegaScheduler {
 public:
  int add_op(const MegaOp& op);
  // n0 x n1 x n2 tasks (a0 slowest); units = what dependants wait for (linear: number of output tiles = n0).
  int add_stage(int type, int op, int n0, int n1, int n2, int dep_stage);
  // policy 0 = round robin, 1 = zig-zag (direction alternates per stage)
  void schedule(int num_sms, int policy);
  const std::vector<MegaTask>& tasks() const { return sorted_; }
  const std::vector<int32_t>& queue_offsets() const { return offsets_; }
  const std::vector<MegaOp>& ops() const { return ops_; }
  int num_stages() const { return static_cast<int>(stages_.size()); }
  int scoreboard_size() const { return static_cast<int>(stages_.size()); }
  std::vector<int> tasks_per_sm() const;

 private:
  struct Stage {
    int type, op, n0, n1, n2, dep, units;
  };
  std::vector<MegaOp> ops_;
  std::vector<Stage> stages_;
  std::vector<MegaTask> sorted_;
  std::vector<int32_t> offsets_;
};

}  // namespace tdb
