// The one Python module of the workspace. Its name is fixed: model_new.py does
// `import cuda_extension` (reference: agent_workdir/binding.cpp:7-10,
// agent_workdir/model_new.py:3). Ops are not listed here; each
// kernels/*_binding.cpp enrols itself through REGISTER_BINDING.
#include <pybind11/pybind11.h>

#include "binding_registry.h"

PYBIND11_MODULE(cuda_extension, m) {
  m.doc() = "B200 (sm_100a) operators behind the agent_workdir binding API";
  BindingRegistry::getInstance().applyBindings(m);
  m.def("registered_ops", []() { return BindingRegistry::getInstance().names(); },
        "Names passed to REGISTER_BINDING, in enrolment order");
}
