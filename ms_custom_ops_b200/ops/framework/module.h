// Operator registry of the B200 plugin.
//
// The reference queues pybind registrations with MS_CUSTOM_OPS_EXTENSION_MODULE
// and replays them when the Python module is created (ops/framework/module.h:30-98).
// Here each operator registers its name and its registered signature (argument
// names, order and defaults); bindings enumerate the registry through the C ABI.
#ifndef MS_CUSTOM_OPS_B200_FRAMEWORK_MODULE_H_
#define MS_CUSTOM_OPS_B200_FRAMEWORK_MODULE_H_

#include <functional>
#include <string>
#include <utility>
#include <vector>

namespace ms_custom_ops {

struct OpEntry {
  std::string name;
  std::string signature;
};

class ModuleRegistry {
 public:
  static ModuleRegistry &Instance() {
    static ModuleRegistry inst;
    return inst;
  }
  void Register(std::string name, std::string signature) {
    for (auto &e : ops_)
      if (e.name == name) return;
    ops_.push_back({std::move(name), std::move(signature)});
  }
  const std::vector<OpEntry> &ops() const { return ops_; }

 private:
  ModuleRegistry() = default;
  std::vector<OpEntry> ops_;
};

#define MS_CUSTOM_OPS_CONCAT_(a, b) a##b
#define MS_CUSTOM_OPS_CONCAT(a, b) MS_CUSTOM_OPS_CONCAT_(a, b)
#define MS_CUSTOM_OPS_REGISTER_OP(op, signature)                                            \
  namespace {                                                                               \
  struct MS_CUSTOM_OPS_CONCAT(op, _registrar) {                                             \
    MS_CUSTOM_OPS_CONCAT(op, _registrar)() {                                                \
      ::ms_custom_ops::ModuleRegistry::Instance().Register(#op, signature);                 \
    }                                                                                       \
  };                                                                                        \
  static MS_CUSTOM_OPS_CONCAT(op, _registrar) MS_CUSTOM_OPS_CONCAT(op, _registrar_instance); \
  }

// Thread-local error slot behind ms_custom_ops_last_error().
void SetLastError(int kind, const std::string &msg);
// Runs `fn`, converting exceptions into (status code, kind, message).
int GuardedCall(const char *op_name, const std::function<int()> &fn);

}  // namespace ms_custom_ops
#endif  // MS_CUSTOM_OPS_B200_FRAMEWORK_MODULE_H_
