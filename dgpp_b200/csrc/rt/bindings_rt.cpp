// Bindings of the remaining runtime components (filled in as components land).
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

namespace py = pybind11;

void bind_more(py::module_& m) { (void)m; }
