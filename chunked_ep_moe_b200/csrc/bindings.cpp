// Python bindings of the sm_100a extension.
#include <torch/extension.h>

#include <ATen/cuda/CUDAContext.h>

#include "gemm/grouped_gemm.cuh"
#include "plan/plan_kernel.cuh"
#include "model/model_ops.h"
#include "runtime/fused_rank.h"
#include "runtime/kernel_runner.h"

namespace {

py::dict plan_layout_dict(int P, int L, int S, int max_slices) {
  const cem::PlanLayout y = cem::make_plan_layout(P, L, S, max_slices);
  py::dict d;
  d["max_mtiles"] = y.max_mtiles;
  d["max_gtiles"] = y.max_gtiles;
  d["max_ptiles"] = y.max_ptiles;
  d["num_ptiles"] = y.off_num_ptiles;
  d["ptiles"] = y.off_ptiles;
  d["send_start"] = y.off_send_start;
  d["seg_start"] = y.off_seg_start;
  d["seg_size"] = y.off_seg_size;
  d["in_start"] = y.off_in_start;
  d["in_size"] = y.off_in_size;
  d["src_send_start"] = y.off_src_send_start;
  d["expert_start"] = y.off_expert_start;
  d["expert_rows"] = y.off_expert_rows;
  d["num_mtiles"] = y.off_num_mtiles;
  d["num_gtiles"] = y.off_num_gtiles;
  d["num_chunks"] = y.off_num_chunks;
  d["mtiles"] = y.off_mtiles;
  d["gtiles"] = y.off_gtiles;
  d["put"] = y.off_put;
  d["total"] = y.total;
  d["tile_m"] = cem::kTileM;
  d["put_chunk_rows"] = cem::kPutChunkRows;
  return d;
}

// CPU restatement of the plan kernel's table build (same code, host-compiled).
torch::Tensor plan_build_host(torch::Tensor counts, int64_t S, int64_t max_slices, int64_t me) {
  TORCH_CHECK(!counts.is_cuda() && counts.scalar_type() == torch::kInt32 && counts.dim() == 3 &&
                  counts.size(0) == counts.size(1) && counts.is_contiguous(),
              "counts must be a contiguous CPU int32 [P, P, L] tensor");
  const int P = static_cast<int>(counts.size(0)), L = static_cast<int>(counts.size(2));
  const cem::PlanLayout y = cem::make_plan_layout(P, L, static_cast<int>(S), static_cast<int>(max_slices));
  torch::Tensor plan = torch::zeros({y.total}, torch::kInt32);
  cem::plan_build_host(counts.data_ptr<int>(), plan.data_ptr<int>(), y, static_cast<int>(me));
  return plan;
}

// The plan kernel itself on a traffic matrix that is already complete in this GPU's memory (no peers to wait for):
// what a rank's kernel computes once every row has landed.
torch::Tensor plan_build_device(torch::Tensor counts, int64_t S, int64_t max_slices, int64_t me) {
  TORCH_CHECK(counts.is_cuda() && counts.scalar_type() == torch::kInt32 && counts.dim() == 3 &&
                  counts.size(0) == counts.size(1) && counts.is_contiguous(),
              "counts must be a contiguous CUDA int32 [P, P, L] tensor");
  const int P = static_cast<int>(counts.size(0)), L = static_cast<int>(counts.size(2));
  TORCH_CHECK(me >= 0 && me < P, "rank out of range");
  cem::PlanKernelParams p{};
  p.lay = cem::make_plan_layout(P, L, static_cast<int>(S), static_cast<int>(max_slices));
  torch::Tensor plan = torch::zeros({p.lay.total}, counts.options());
  torch::Tensor mine = counts[me].contiguous();
  p.me = static_cast<int>(me);
  p.my_counts = mine.data_ptr<int>();
  p.counts = counts.data_ptr<int>();
  p.plan = plan.data_ptr<int>();
  cem::launch_plan_build(p, at::cuda::getCurrentCUDAStream());
  return plan;
}

int64_t arena_bytes(int P, int L, int S, int D, int tk_cap, bool fp8) {
  return static_cast<int64_t>(cem::make_arena_layout(P, L, S, D, tk_cap, fp8).total);
}

py::dict arena_layout_dict(int P, int L, int S, int D, int tk_cap, bool fp8) {
  const cem::ArenaLayout a = cem::make_arena_layout(P, L, S, D, tk_cap, fp8);
  py::dict d;
  d["xbuf"] = a.xbuf; d["gbuf"] = a.gbuf; d["wbuf"] = a.wbuf; d["xq"] = a.xq; d["gq"] = a.gq; d["xs"] = a.xs;
  d["gs"] = a.gs; d["ret"] = a.ret; d["dw_rows"] = a.dw_rows; d["arrive"] = a.arrive; d["credit"] = a.credit;
  d["ret_count"] = a.ret_count; d["traffic"] = a.traffic; d["traffic_flags"] = a.traffic_flags; d["total"] = a.total;
  return d;
}

void wait_probe(torch::Tensor flag, int64_t target, int64_t spin_limit, torch::Tensor status) {
  TORCH_CHECK(flag.is_cuda() && flag.scalar_type() == torch::kInt32 && status.is_cuda() &&
                  status.scalar_type() == torch::kInt32 && status.numel() >= 8,
              "flag and status must be CUDA int32 tensors (status: 8 ints)");
  cem::launch_wait_probe(reinterpret_cast<const uint32_t*>(flag.data_ptr()), static_cast<uint32_t>(target),
                         static_cast<uint32_t>(spin_limit), reinterpret_cast<cem::StatusBlock*>(status.data_ptr()),
                         at::cuda::getCurrentCUDAStream().stream());
}

}  // namespace

PYBIND11_MODULE(TORCH_EXTENSION_NAME, m) {
  m.doc() = "chunked expert-parallel MoE: sm_100a kernels and runtime";
  m.def("plan_layout", &plan_layout_dict, "offsets of the per-pass plan buffer");
  m.def("plan_build_host", &plan_build_host, "host build of the per-pass plan tables (CPU tests)");
  m.def("plan_build_device", &plan_build_device, "the plan kernel on a complete traffic matrix (GPU tests)");
  m.def("arena_bytes", &arena_bytes, "size of one rank's symmetric arena");
  m.def("arena_alloc", &cem::arena_alloc);
  m.def("arena_free", &cem::arena_free);
  m.def("arena_export", &cem::arena_export);
  m.def("arena_import", &cem::arena_import);
  m.def("arena_close", &cem::arena_close);
  m.def("arena_zero", &cem::arena_zero);
  m.def("arena_fill", &cem::arena_fill, "cudaMemset of a byte range (tests poison data buffers with NaN patterns)");
  m.def("arena_layout", &arena_layout_dict, "byte offsets inside one rank's symmetric arena");
  m.def("arena_read_i32", &cem::arena_read_i32, "device synchronise + copy int32 values of an arena to the host");
  m.attr("gemm_smem_bytes") = cem::kGemmSmemBytes;
  m.def("pair_grid_used", []() { return cem::g_pair_grid_used; }, "grid of the last CTA-pair GEMM launch");
  m.def("wait_probe", &wait_probe, "bounded-wait self test kernel");
  m.def("format_status", &cem::format_status, "text of a recorded status block");
  m.def("add_rms_norm_fwd", &cem::add_rms_norm_fwd, "s = x + delta, y = RMSNorm(s) * w -> (s, y, rstd)");
  m.def("add_rms_norm_bwd", &cem::add_rms_norm_bwd, "-> (ds, dweight)");
  m.def("rope_qkv_fwd", &cem::rope_qkv_fwd, "qkv [B,S,3,H,hd] -> rotated q, k and v as [B,H,S,hd]");
  m.def("rope_qkv_bwd", &cem::rope_qkv_bwd, "gradients of q, k, v -> gradient of qkv");
  m.def("cross_entropy_fwd", &cem::cross_entropy_fwd, "bf16 logits -> (loss per row, log-sum-exp per row)");
  m.def("cross_entropy_bwd", &cem::cross_entropy_bwd, "-> bf16 gradient of the logits");
  m.def("dense_swiglu_fwd", &cem::dense_swiglu_fwd, "[gate | up] -> silu(gate) * up");
  m.def("dense_swiglu_bwd", &cem::dense_swiglu_bwd, "-> gradient of [gate | up]");
  m.def("router_fwd", &cem::router_fwd, "fp32 logits, bias -> (ids, weights, counts, per-block score sums)");
  m.def("router_bwd", &cem::router_bwd, "-> fp32 gradient of the logits");
  py::class_<cem::KernelRunner>(m, "KernelRunner")
      .def(py::init<int, int, int, int, bool>(), py::arg("L"), py::arg("S"), py::arg("stripe"), py::arg("num_sms"),
           py::arg("cta_pairs") = false)
      .def("set_groups", &cem::KernelRunner::set_groups)
      .def("gmm_swiglu", &cem::KernelRunner::gmm_swiglu, py::arg("x"), py::arg("w_up"), py::arg("act"),
           py::arg("h") = py::none())
      .def("gmm", &cem::KernelRunner::gmm)
      .def("gmm_down_dw", &cem::KernelRunner::gmm_down_dw)
      .def("gmm_dswiglu", &cem::KernelRunner::gmm_dswiglu)
      .def("tgmm", &cem::KernelRunner::tgmm)
      .def("check_status", &cem::KernelRunner::check_status);
  py::class_<cem::FusedRank>(m, "FusedRank")
      .def(py::init<int, int, int, int, int, int, int, int, int, int, int, bool, int64_t, std::vector<int64_t>, bool,
                    int64_t, int, bool, bool>(),
           py::arg("P"), py::arg("L"), py::arg("me"), py::arg("S"), py::arg("D"), py::arg("F"), py::arg("K"),
           py::arg("stripe"), py::arg("tk_cap"), py::arg("max_slices"), py::arg("num_sms"), py::arg("fp8"),
           py::arg("arena"), py::arg("peer_arenas"), py::arg("use_comm_stream"), py::arg("spin_limit"),
           py::arg("put_blocks"), py::arg("cta_pairs") = true, py::arg("tgmm_pairs") = true)
      .def("begin_forward", &cem::FusedRank::begin_forward)
      .def("begin_forward_async", &cem::FusedRank::begin_forward_async)
      .def("resolve_slices", &cem::FusedRank::resolve_slices)
      .def("set_pass_slices", &cem::FusedRank::set_pass_slices)
      .def("set_mbar_limit_us", &cem::FusedRank::set_mbar_limit_us)
      .def("sort_only", &cem::FusedRank::sort_only)
      .def("begin_backward", &cem::FusedRank::begin_backward, py::arg("plan"), py::arg("known_slices") = -1,
           py::arg("known_rows") = -1)
      .def("put", &cem::FusedRank::put)
      .def("compute_forward", &cem::FusedRank::compute_forward)
      .def("compute_backward", &cem::FusedRank::compute_backward)
      .def("finish_forward", &cem::FusedRank::finish_forward)
      .def("finish_backward", &cem::FusedRank::finish_backward)
      .def("check_status", &cem::FusedRank::check_status)
      .def("plan_header", &cem::FusedRank::plan_header)
      .def("plan_ints", &cem::FusedRank::plan_ints)
      .def("launches", &cem::FusedRank::launches)
      .def("set_pipeline_counters", &cem::FusedRank::set_pipeline_counters, py::arg("counters") = py::none())
      .def("act", &cem::FusedRank::act)
      .def("h", &cem::FusedRank::h)
      .def("dh", &cem::FusedRank::dh)
      .def("dy", &cem::FusedRank::dy);
}
