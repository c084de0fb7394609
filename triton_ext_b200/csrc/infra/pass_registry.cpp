// Process-wide registry of extension passes behind the four plugin entry points declared in
// triton_ext_plugin.h. One copy per process: every extension library links this shared library, the
// way the reference links TritonExtPassInfra PUBLIC (pass/LoopSplit/CMakeLists.txt:25-26).
//
// Behaviour follows infra/pass/TritonExtPassInfra.cpp:7-52 of the reference: names map to an
// "add to pipeline" callback and a "register" callback; lookups of unknown names and a null count
// pointer fail with TP_GENERIC_FAILURE; names are borrowed from the extension. Enumeration fills
// every slot (the reference leaves all names in slot 0) and the tables are mutex-guarded.
#include <cstring>
#include <mutex>
#include <string>
#include <vector>

#include "triton_ext_plugin.h"

namespace {

struct Entry {
  const char *name;  // borrowed: points into the extension library's read-only data
  TritonExtRegisterPassFunc register_fn;
  TritonExtAddPassFunc add_fn;
};

struct Registry {
  std::mutex mu;
  std::vector<Entry> entries;  // load order == enumeration order

  Entry *find(const char *name) {
    for (Entry &e : entries)
      if (std::strcmp(e.name, name) == 0) return &e;
    return nullptr;
  }
};

Registry &registry() {
  // Constructed on first use: extension static initialisers may run before this library's own.
  static Registry *r = new Registry();
  return *r;
}

}  // namespace

TRITON_PLUGIN_API
TritonExtLoadPass(const char *passName, TritonExtRegisterPassFunc registerFunc, TritonExtAddPassFunc addFunc) {
  if (!passName || !registerFunc || !addFunc) return TP_GENERIC_FAILURE;
  Registry &r = registry();
  std::lock_guard<std::mutex> lock(r.mu);
  if (Entry *e = r.find(passName)) {  // loading the same name again replaces the callbacks
    e->name = passName;
    e->register_fn = registerFunc;
    e->add_fn = addFunc;
  } else {
    r.entries.push_back(Entry{passName, registerFunc, addFunc});
  }
  return TP_SUCCESS;
}

TRITON_PLUGIN_API
tritonAddPluginPass(TritonExtPassManagerRef pm, const char *passName) {
  if (!passName || !pm) return TP_GENERIC_FAILURE;
  TritonExtAddPassFunc fn = nullptr;
  {
    Registry &r = registry();
    std::lock_guard<std::mutex> lock(r.mu);
    if (Entry *e = r.find(passName)) fn = e->add_fn;
  }
  if (!fn) return TP_GENERIC_FAILURE;
  fn(pm);  // outside the lock: the callback may itself consult the registry
  return TP_SUCCESS;
}

TRITON_PLUGIN_API
tritonRegisterPluginPass(const char *passName) {
  if (!passName) return TP_GENERIC_FAILURE;
  TritonExtRegisterPassFunc fn = nullptr;
  {
    Registry &r = registry();
    std::lock_guard<std::mutex> lock(r.mu);
    if (Entry *e = r.find(passName)) fn = e->register_fn;
  }
  if (!fn) return TP_GENERIC_FAILURE;
  fn();
  return TP_SUCCESS;
}

TRITON_PLUGIN_API
tritonEnumeratePluginPasses(uint32_t *passCount, const char **passNames) {
  if (!passCount) return TP_GENERIC_FAILURE;
  Registry &r = registry();
  std::lock_guard<std::mutex> lock(r.mu);
  *passCount = static_cast<uint32_t>(r.entries.size());
  if (!passNames) return TP_SUCCESS;
  uint32_t i = 0;
  for (const Entry &e : r.entries) passNames[i++] = e.name;
  return TP_SUCCESS;
}
