// function_map_<p>.so: the per-partition plugin the Cerium runtime loads
// (CeriumFunction::load_function_map, cerium/runtime/execution/function.cpp:144-177).
//
// The runtime resolves two asm-labelled getters in it, __GET_FUNCTION_MAP__ and
// __GET_FUNCTION_MAP_CUGRAPH__ (generated today by KernelFusionContext::write_function_map,
// cerium/compiler/backend/cuda_kernel.cc:1972-2074), each returning a map kernel id -> host launcher.
// This shim is a few lines on purpose: it finds its own file name <dir>/function_map_<p>.so, names
// the partition's records file <dir>/functions<p> (and the generated plugin, when it was kept beside
// it as function_map_<p>.orig.so), and hands both to libcerium_b200.so, which owns the launchers and
// keeps one pair of maps per records file.
//
// Install one COPY of the built shim per partition.  The runtime loads every partition's plugin into
// one process; links to a single file would be folded into one loaded object by the dynamic loader
// and every partition would then see the first one's path.  The shim is linked against
// libcerium_b200.so, so a context bound through the library (cerium_function_map_bind) by the host
// program is the one the launchers find.
#include <dlfcn.h>

#include <cstdint>
#include <fstream>
#include <stdexcept>
#include <string>
#include <unordered_map>

extern "C" {
const void* cerium_function_map_get(const char* functions_path, const char* generated_plugin_path, int cugraph);
const char* cerium_function_map_error(void);
}

namespace {

using FunctionMapType = std::unordered_map<uint32_t, void*>;

const FunctionMapType& partition_map(int cugraph) {
  Dl_info info{};
  if (!dladdr((void*)&partition_map, &info) || !info.dli_fname)
    throw std::runtime_error("cerium_b200 plugin: cannot find the path of the plugin");
  const std::string self = info.dli_fname;
  const size_t slash = self.find_last_of('/');
  const std::string dir = slash == std::string::npos ? std::string(".") : self.substr(0, slash);
  const std::string base = slash == std::string::npos ? self : self.substr(slash + 1);
  const std::string prefix = "function_map_", suffix = ".so";
  if (base.size() <= prefix.size() + suffix.size() || base.compare(0, prefix.size(), prefix) != 0 ||
      base.compare(base.size() - suffix.size(), suffix.size(), suffix) != 0)
    throw std::runtime_error("cerium_b200 plugin: loaded as '" + base + "', not as function_map_<p>.so");
  const std::string p = base.substr(prefix.size(), base.size() - prefix.size() - suffix.size());
  const std::string functions = dir + "/functions" + p;
  const std::string orig = dir + "/function_map_" + p + ".orig.so";
  const bool have_orig = std::ifstream(orig).is_open();
  const void* m = cerium_function_map_get(functions.c_str(), have_orig ? orig.c_str() : nullptr, cugraph);
  if (!m) throw std::runtime_error(std::string("cerium_b200 plugin (partition ") + p + "): " + cerium_function_map_error());
  return *static_cast<const FunctionMapType*>(m);
}

}  // namespace

__attribute__((visibility("default"))) const FunctionMapType& cerium_b200_get_function_map() asm("__GET_FUNCTION_MAP__");
__attribute__((visibility("default"))) const FunctionMapType& cerium_b200_get_function_map_cugraph() asm(
    "__GET_FUNCTION_MAP_CUGRAPH__");
const FunctionMapType& cerium_b200_get_function_map() { return partition_map(0); }
const FunctionMapType& cerium_b200_get_function_map_cugraph() { return partition_map(1); }
