// Task-graph scheduler of the decode megakernel (see tdb/mega.h).
#include <algorithm>
#include <stdexcept>

#include "tdb/mega.h"

namespace tdb {

int MegaScheduler::add_op(const MegaOp& op) {
  ops_.push_back(op);
  return static_cast<int>(ops_.size()) - 1;
}

int MegaScheduler::add_stage(int type, int op, int n0, int n1, int n2, int dep_stage) {
  if (op < 0 || op >= static_cast<int>(ops_.size())) throw std::runtime_error("mega: bad op index");
  if (dep_stage >= static_cast<int>(stages_.size())) throw std::runtime_error("mega: a stage may only depend on an earlier stage");
  if (n0 < 1 || n1 < 1 || n2 < 1) throw std::runtime_error("mega: empty stage");
  Stage s;
  s.type = type; s.op = op; s.n0 = n0; s.n1 = n1; s.n2 = n2; s.dep = dep_stage;
  s.units = (type == kTaskLinear) ? n0 : n0 * n1 * n2;
  stages_.push_back(s);
  return static_cast<int>(stages_.size()) - 1;
}

void MegaScheduler::schedule(int num_sms, int policy) {
  if (num_sms < 1) throw std::runtime_error("mega: need at least one SM");
  std::vector<std::vector<MegaTask>> q(num_sms);
  int cursor = 0;
  for (int si = 0; si < static_cast<int>(stages_.size()); ++si) {
    const Stage& s = stages_[si];
    const int n = s.n0 * s.n1 * s.n2;
    for (int j = 0; j < n; ++j) {
      MegaTask t{};
      t.type = s.type;
      t.dep_idx = s.dep;
      t.dep_need = s.dep >= 0 ? stages_[s.dep].units : 0;
      t.out_idx = si;
      t.op = s.op;
      t.a0 = j / (s.n1 * s.n2);
      t.a1 = (j / s.n2) % s.n1;
      t.a2 = j % s.n2;
      int sm = (cursor + j) % num_sms;
      if (policy == 1 && (si & 1)) sm = num_sms - 1 - sm;
      q[sm].push_back(t);
    }
    cursor = (cursor + n) % num_sms;
  }
  sorted_.clear();
  offsets_.assign(num_sms + 1, 0);
  for (int sm = 0; sm < num_sms; ++sm) {
    offsets_[sm] = static_cast<int32_t>(sorted_.size());
    sorted_.insert(sorted_.end(), q[sm].begin(), q[sm].end());
  }
  offsets_[num_sms] = static_cast<int32_t>(sorted_.size());
}

std::vector<int> MegaScheduler::tasks_per_sm() const {
  std::vector<int> r;
  for (size_t i = 0; i + 1 < offsets_.size(); ++i) r.push_back(offsets_[i + 1] - offsets_[i]);
  return r;
}

}  // namespace tdb
