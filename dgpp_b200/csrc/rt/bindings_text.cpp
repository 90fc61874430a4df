// Bindings of the text stack (tokenizer, chat template).
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

namespace py = pybind11;

void bind_text(py::module_& m) { (void)m; }
