#include <pybind11/pybind11.h>
namespace py = pybind11;
void bind_symm(py::module_& m) {}
