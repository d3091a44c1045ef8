// Python bindings of the host-side serving runtime (page allocator, radix tree).
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include "radix.h"

namespace py = pybind11;

void register_runtime(py::module_& m) {
  py::class_<hb::PageAllocator>(m, "PageAllocator")
      .def(py::init<int>(), py::arg("num_pages"))
      .def("alloc",
           [](hb::PageAllocator& a, int n) -> py::object {
             std::vector<int32_t> out;
             if (!a.alloc(n, out)) return py::none();
             return py::cast(out);
           })
      .def("free", &hb::PageAllocator::free)
      .def("available", &hb::PageAllocator::available)
      .def("capacity", &hb::PageAllocator::capacity)
      .def("clear", &hb::PageAllocator::clear);

  py::class_<hb::RadixTree>(m, "RadixTree")
      .def(py::init<int>(), py::arg("page_size"))
      .def("reset", &hb::RadixTree::reset)
      .def("match_prefix",
           [](hb::RadixTree& t, const std::vector<int32_t>& tokens) {
             std::vector<int32_t> pages;
             const int64_t node = t.match_prefix(tokens, pages);
             return py::make_tuple(pages, node);
           })
      .def("insert", &hb::RadixTree::insert)
      .def("inc_lock_ref", &hb::RadixTree::inc_lock_ref)
      .def("dec_lock_ref", &hb::RadixTree::dec_lock_ref)
      .def("evict",
           [](hb::RadixTree& t, int n) {
             std::vector<int32_t> freed;
             t.evict(n, freed);
             return freed;
           })
      .def_property_readonly("evictable_pages", &hb::RadixTree::evictable_pages)
      .def_property_readonly("protected_pages", &hb::RadixTree::protected_pages)
      .def("total_pages", &hb::RadixTree::total_pages)
      .def("node_count", &hb::RadixTree::node_count)
      .def("sanity_check", &hb::RadixTree::sanity_check);
}
