// pybind11 surface of the page-id pool: BlockPool(num_blocks), allocate, free and
// the read-only properties num_blocks / num_free / num_used / utilization, as in
// the reference's module (core/python/bindings.cpp:8-22).  std::runtime_error
// arrives in Python as RuntimeError, std::invalid_argument as ValueError.
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include "block_pool.h"

namespace py = pybind11;

PYBIND11_MODULE(distie_b200_core, m) {
  m.doc() = "Page-id pool of the distie_b200 paged cache";
  py::class_<distie_b200::BlockPool>(m, "BlockPool")
      .def(py::init<std::size_t>(), py::arg("num_blocks"))
      .def("allocate", &distie_b200::BlockPool::Allocate, py::arg("count"))
      .def("free", &distie_b200::BlockPool::Free, py::arg("block_ids"))
      .def_property_readonly("num_blocks", &distie_b200::BlockPool::num_blocks)
      .def_property_readonly("num_free", &distie_b200::BlockPool::num_free)
      .def_property_readonly("num_used", &distie_b200::BlockPool::num_used)
      .def_property_readonly("utilization", &distie_b200::BlockPool::utilization);
}
