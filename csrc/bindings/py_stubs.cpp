// Placeholders until the corresponding components are linked in.
#include <pybind11/pybind11.h>
namespace py = pybind11;
void bind_ops(py::module_&) {}
