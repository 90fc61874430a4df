// pybind11 surface of the native host runtime.
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include "rt/paged_blocks.h"

namespace py = pybind11;

void bind_more(py::module_& m);  // defined in bindings_rt.cpp when present

PYBIND11_MODULE(_dgpp_rt, m) {
  m.doc() = "dgpp_b200 native host runtime";
  py::class_<dgpp::PagedBlockTable>(m, "PagedBlockTable")
      .def(py::init<int>())
      .def("num_blocks", &dgpp::PagedBlockTable::num_blocks)
      .def("free_count", &dgpp::PagedBlockTable::free_count)
      .def("alloc", &dgpp::PagedBlockTable::alloc)
      .def("retain", &dgpp::PagedBlockTable::retain)
      .def("release", &dgpp::PagedBlockTable::release)
      .def("refcount", &dgpp::PagedBlockTable::refcount)
      .def("generation", &dgpp::PagedBlockTable::generation);
  bind_more(m);
}
