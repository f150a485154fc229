// Bindings for the host-side components that are not part of the step loop (tokenizer,
// detokenizer, loaders, structured output, KV offload). Each component registers itself
// here as it is added.
#include <pybind11/pybind11.h>
namespace py = pybind11;

void bind_tokenizer(py::module_& m) __attribute__((weak));
void bind_loaders(py::module_& m) __attribute__((weak));
void bind_structured(py::module_& m) __attribute__((weak));
void bind_offload(py::module_& m) __attribute__((weak));
void bind_cpu_backend(py::module_& m) __attribute__((weak));
void bind_frontend(py::module_& m) __attribute__((weak));
void bind_parallel(py::module_& m) __attribute__((weak));

void bind_extras(py::module_& m) {
  if (bind_tokenizer) bind_tokenizer(m);
  if (bind_loaders) bind_loaders(m);
  if (bind_structured) bind_structured(m);
  if (bind_offload) bind_offload(m);
  if (bind_cpu_backend) bind_cpu_backend(m);
  if (bind_frontend) bind_frontend(m);
  if (bind_parallel) bind_parallel(m);
}
