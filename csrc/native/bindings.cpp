// pybind11 module `_pb200_native`: one sub-module per systems component.
#include <pybind11/pybind11.h>

#include "common.hpp"

namespace py = pybind11;

void bind_loader(py::module_& m);
void bind_ckpt(py::module_& m);
void bind_control(py::module_& m);
void bind_obs(py::module_& m);
void bind_harness_core(py::module_& m);
void bind_harness_queue(py::module_& m);
void bind_harness_control(py::module_& m);
void bind_harness_lab(py::module_& m);
void bind_harness_faults(py::module_& m);
void bind_rl_core(py::module_& m);
void bind_rl_envs(py::module_& m);
void bind_data_pipeline(py::module_& m);
void bind_rl_tasks(py::module_& m);
void bind_synth(py::module_& m);
void bind_contracts(py::module_& m);
void bind_verify_stages(py::module_& m);

PYBIND11_MODULE(_pb200_native, m) {
  m.doc() = "C++ systems components of prometheus_b200 (loader, checkpoints, control, ...)";
  // NativeError carries `.kind` (e.g. "NotFound", "HashMismatch") next to the message.
  static py::exception<pbn::Error> native_error(m, "NativeError", PyExc_RuntimeError);
  py::register_exception_translator([](std::exception_ptr p) {
    try {
      if (p) std::rethrow_exception(p);
    } catch (const pbn::Error& e) {
      py::object exc = py::handle(native_error.ptr())(std::string(e.what()));
      exc.attr("kind") = e.kind;
      PyErr_SetObject(native_error.ptr(), exc.ptr());
    }
  });
  auto loader = m.def_submodule("loader", "deterministic packing / shuffle / resumable loader");
  bind_loader(loader);
  auto ckpt = m.def_submodule("ckpt", "content-addressed sharded checkpoints");
  bind_ckpt(ckpt);
  auto control = m.def_submodule("control", "elastic controller, rungs, scaling-law fit");
  bind_control(control);
  auto obs = m.def_submodule("obs", "metrics, tracing, run registry, spike log");
  bind_obs(obs);
  bind_harness_core(m);
  bind_harness_queue(m);
  bind_harness_control(m);
  bind_harness_lab(m);
  bind_harness_faults(m);
  bind_rl_core(m);
  bind_rl_envs(m);
  bind_data_pipeline(m);
  bind_rl_tasks(m);
  bind_synth(m);
  bind_contracts(m);
  bind_verify_stages(m);
}
