// Op registration for the `cuda_extension` Python module.
//
// Same public surface as the reference workspace header
// (agent_workdir/binding_registry.h:15-49): a process-wide BindingRegistry,
// a BindingRegistrar whose constructor enrols one callback, and the
// REGISTER_BINDING(name, func) macro that a `*_binding.cpp` file ends with.
// A binding file written for the reference workspace compiles against this
// header unchanged.
//
// Differences that do not alter behaviour for a well-formed workspace:
//   * enrolling the same op name twice is rejected at module import with a
//     std::runtime_error naming the op (the reference silently defines the
//     second pybind overload over the first);
//   * names() lists what was enrolled, which the tests use to check that every
//     launcher declared in include/cuda_agent_b200.h has a Python binding.
#pragma once

#include <functional>
#include <stdexcept>
#include <string>
#include <utility>
#include <vector>

#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

class BindingRegistry {
 public:
  using BindingFunction = std::function<void(pybind11::module&)>;

  // Function-local static: constructed on first use, so registrars in other
  // translation units may run before or after any other static initialiser.
  static BindingRegistry& getInstance() {
    static BindingRegistry the_registry;
    return the_registry;
  }

  void registerBinding(const std::string& name, BindingFunction func) {
    for (const Entry& e : entries_) {
      if (e.first == name) {
        duplicate_ = name;  // reported when the module is imported
        return;
      }
    }
    entries_.emplace_back(name, std::move(func));
  }

  // Called once from PYBIND11_MODULE; runs every enrolled callback on `m`.
  void applyBindings(pybind11::module& m) {
    if (!duplicate_.empty()) {
      throw std::runtime_error("REGISTER_BINDING: op '" + duplicate_ + "' registered twice");
    }
    for (Entry& e : entries_) e.second(m);
  }

  std::vector<std::string> names() const {
    std::vector<std::string> out;
    out.reserve(entries_.size());
    for (const Entry& e : entries_) out.push_back(e.first);
    return out;
  }

  BindingRegistry(const BindingRegistry&) = delete;
  BindingRegistry& operator=(const BindingRegistry&) = delete;

 private:
  using Entry = std::pair<std::string, BindingFunction>;
  BindingRegistry() = default;
  std::vector<Entry> entries_;
  std::string duplicate_;
};

// One static instance per binding file does the enrolment at load time.
class BindingRegistrar {
 public:
  BindingRegistrar(const std::string& name, BindingRegistry::BindingFunction func) {
    BindingRegistry::getInstance().registerBinding(name, std::move(func));
  }
};

#define REGISTER_BINDING(name, func) \
  static BindingRegistrar _registrar_##name(#name, [](pybind11::module& m) { func(m); })
