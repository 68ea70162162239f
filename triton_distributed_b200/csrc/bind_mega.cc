// Python bindings of the megakernel scheduler and launcher.
#include <ATen/cuda/CUDAContext.h>
#include <c10/cuda/CUDAGuard.h>
#include <torch/extension.h>

#include "tdb/mega.h"
#include "tdb/symm_heap.h"

namespace py = pybind11;
using tdb::MegaScheduler;
using tdb::SymmHeap;

namespace {

cudaStream_t cur_stream() { return at::cuda::getCurrentCUDAStream().stream(); }
void check_cuda(cudaError_t e, const char* what) { TORCH_CHECK(e == cudaSuccess, what, ": ", cudaGetErrorString(e)); }

int add_op(MegaScheduler& s, const std::vector<uint64_t>& ptrs, const std::vector<int32_t>& ints,
           const std::vector<float>& floats) {
  TORCH_CHECK(ptrs.size() <= 8 && ints.size() <= 12 && floats.size() <= 4, "mega op: too many fields");
  tdb::MegaOp op;
  std::memset(&op, 0, sizeof(op));
  for (size_t i = 0; i < ptrs.size(); ++i) op.p[i] = reinterpret_cast<void*>(ptrs[i]);
  for (size_t i = 0; i < ints.size(); ++i) op.i[i] = ints[i];
  for (size_t i = 0; i < floats.size(); ++i) op.f[i] = floats[i];
  return s.add_op(op);
}

// byte images to upload
at::Tensor tasks_tensor(MegaScheduler& s) {
  const auto& t = s.tasks();
  at::Tensor out = at::empty({static_cast<int64_t>(t.size()), 16}, at::kInt);
  if (!t.empty()) std::memcpy(out.data_ptr(), t.data(), t.size() * sizeof(tdb::MegaTask));
  return out;
}
at::Tensor offsets_tensor(MegaScheduler& s) {
  const auto& o = s.queue_offsets();
  at::Tensor out = at::empty({static_cast<int64_t>(o.size())}, at::kInt);
  std::memcpy(out.data_ptr(), o.data(), o.size() * sizeof(int32_t));
  return out;
}
at::Tensor ops_tensor(MegaScheduler& s) {
  const auto& o = s.ops();
  at::Tensor out = at::empty({static_cast<int64_t>(o.size()), static_cast<int64_t>(sizeof(tdb::MegaOp))}, at::kByte);
  if (!o.empty()) std::memcpy(out.data_ptr(), o.data(), o.size() * sizeof(tdb::MegaOp));
  return out;
}

// 2-D K-major tensor map [rows, cols] with box [box_rows, 64], 128-byte swizzle -> 128 bytes (uint8 CPU tensor)
at::Tensor make_tensor_map(const at::Tensor& t, int64_t box_rows) {
  TORCH_CHECK(t.is_cuda() && t.dim() == 2 && t.stride(1) == 1 && t.scalar_type() == at::kBFloat16, "tensor map: bf16 [rows, cols]");
  tdb::TensorMap m;
  const int r = tdb::encode_tensor_map_2d(&m, t.data_ptr(), tdb::kBF16, t.size(0), t.size(1), t.stride(0) * 2, box_rows, 64, 128);
  TORCH_CHECK(r == 0, "cuTensorMapEncodeTiled failed with code ", r);
  at::Tensor out = at::empty({128}, at::kByte);
  std::memcpy(out.data_ptr(), m.bytes, 128);
  return out;
}

void mega_launch(SymmHeap* h, const at::Tensor& tasks, const at::Tensor& offsets, const at::Tensor& ops, const at::Tensor& tmaps,
                 at::Tensor& scoreboard, at::Tensor& acc, at::Tensor& counters, at::Tensor& ctx, int64_t batch, int64_t grid,
                 bool use_multimem, c10::optional<at::Tensor> profile_buf, double timeout_s) {
  c10::cuda::CUDAGuard guard(tasks.device());
  tdb::MegaLaunchArgs a;
  a.tasks = reinterpret_cast<const tdb::MegaTask*>(tasks.data_ptr());
  a.queue_offsets = offsets.data_ptr<int32_t>();
  a.ops = reinterpret_cast<const tdb::MegaOp*>(ops.data_ptr());
  a.tmaps = tmaps.data_ptr();
  TORCH_CHECK((reinterpret_cast<uintptr_t>(a.tmaps) & 63u) == 0, "tensor maps must be 64-byte aligned");
  a.scoreboard = scoreboard.data_ptr<int32_t>();
  a.scoreboard_size = scoreboard.numel();
  a.acc = acc.data_ptr<float>();
  a.counters = reinterpret_cast<uint32_t*>(counters.data_ptr());
  a.ctx = reinterpret_cast<tdb::CtxDev*>(ctx.data_ptr());
  if (h != nullptr) {
    a.symm = h->info(static_cast<uint64_t>(timeout_s * 1e9));
  } else {
    std::memset(&a.symm, 0, sizeof(a.symm));
    a.symm.world = 1;
    a.symm.timeout_ns = static_cast<uint64_t>(timeout_s * 1e9);
  }
  a.batch = batch;
  a.grid = grid;
  a.use_multimem = use_multimem ? 1 : 0;
  a.profile_buf = profile_buf.has_value() ? profile_buf->data_ptr() : nullptr;
  check_cuda(tdb::launch_megakernel(a, cur_stream()), "launch_megakernel");
}

}  // namespace

void bind_mega(py::module_& m) {
  py::class_<MegaScheduler>(m, "MegaScheduler")
      .def(py::init<>())
      .def("add_op", &add_op)
      .def("add_stage", &MegaScheduler::add_stage)
      .def("schedule", &MegaScheduler::schedule)
      .def("tasks_tensor", &tasks_tensor)
      .def("offsets_tensor", &offsets_tensor)
      .def("ops_tensor", &ops_tensor)
      .def("tasks_per_sm", &MegaScheduler::tasks_per_sm)
      .def_property_readonly("num_stages", &MegaScheduler::num_stages)
      .def_property_readonly("scoreboard_size", &MegaScheduler::scoreboard_size);
  m.def("make_tensor_map", &make_tensor_map);
  m.def("mega_launch", &mega_launch);
  m.def("megakernel_mpad", &tdb::megakernel_mpad);
}
