// `nexus_b200._native`: the host-side native runtime (archive codecs, checksums, allocator and
// planner, profiler, CPU oracles, environments, the rendezvous store and the watchdog scan).  Each translation unit registers its own bindings.
#include <pybind11/pybind11.h>

namespace py = pybind11;

void bind_nxs2(py::module_& m);
void bind_nxs3(py::module_& m);
void bind_runtime(py::module_& m);
void bind_cpu_kernels(py::module_& m);
void bind_envs(py::module_& m);
void bind_device_allocator(py::module_& m);
void bind_store(py::module_& m);
void bind_moe_ref(py::module_& m);
void bind_estimate(py::module_& m);
void bind_dlpack(py::module_& m);
void bind_token_data(py::module_& m);
void bind_kv_sched(py::module_& m);
void bind_lowp(py::module_& m);
void bind_fused_train_cpu(py::module_& m);
void bind_moe_route(py::module_& m);
void bind_pipeline_sched(py::module_& m);
void bind_rl_core(py::module_& m);
void bind_tb_events(py::module_& m);

PYBIND11_MODULE(_native, m) {
  m.doc() = "nexus_b200 native host runtime";
  bind_nxs2(m);
  bind_nxs3(m);
  bind_runtime(m);
  bind_cpu_kernels(m);
  bind_envs(m);
  bind_device_allocator(m);
  bind_store(m);
  bind_moe_ref(m);
  bind_estimate(m);
  bind_dlpack(m);
  bind_token_data(m);
  bind_kv_sched(m);
  bind_lowp(m);
  bind_fused_train_cpu(m);
  bind_moe_route(m);
  bind_pipeline_sched(m);
  bind_rl_core(m);
  bind_tb_events(m);
}
