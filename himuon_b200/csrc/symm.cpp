#include "symm.h"
namespace himuon {
void bind_symm(pybind11::module_& m) { (void)m; }
}  // namespace himuon
