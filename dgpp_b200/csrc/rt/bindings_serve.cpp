// Bindings of the sampler oracle, grammars and HTTP server.
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

namespace py = pybind11;

void bind_serve(py::module_& m) { (void)m; }
