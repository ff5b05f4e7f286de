// Bindings for routing, communication and the symmetric-memory runtime.
#include <torch/extension.h>

void register_more(pybind11::module_& m) { (void)m; }
