// Symmetric (peer-mapped) device memory and the collective kernels that run over it.
#pragma once
#include <pybind11/pybind11.h>
namespace himuon {
void bind_symm(pybind11::module_& m);
}
