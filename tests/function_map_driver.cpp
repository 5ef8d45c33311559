// Loads a function_map_<p>.so the way the reference runtime does (dlopen, dlsym of the two asm-labelled
// getters, call; cerium/runtime/execution/function.cpp:144-177) and prints the maps it returns, one
// "<stream|graph> <id> <launcher address>" line per entry.  TEST INFRASTRUCTURE: built by
// tests/test_function_map.py with g++; needs no GPU (the getters only build the maps).
#include <dlfcn.h>

#include <cstdint>
#include <cstdio>
#include <exception>
#include <unordered_map>

typedef std::unordered_map<uint32_t, void*> FunctionMapType;
typedef const FunctionMapType& (*map_function_t)();

int main(int argc, char** argv) {
  if (argc < 2) return 2;
  void* h = dlopen(argv[1], RTLD_LAZY);
  if (!h) {
    std::fprintf(stderr, "dlopen: %s\n", dlerror());
    return 3;
  }
  const char* names[2] = {"__GET_FUNCTION_MAP__", "__GET_FUNCTION_MAP_CUGRAPH__"};
  const char* tags[2] = {"stream", "graph"};
  for (int k = 0; k < 2; k++) {
    map_function_t get = (map_function_t)dlsym(h, names[k]);
    if (!get) {
      std::fprintf(stderr, "dlsym %s: %s\n", names[k], dlerror());
      return 4;
    }
    try {
      const FunctionMapType& m = get();
      for (const auto& kv : m) std::printf("%s %u %p\n", tags[k], kv.first, kv.second);
    } catch (const std::exception& e) {
      std::printf("error %s\n", e.what());
      return 5;
    }
  }
  typedef void* (*launcher_t)(const char*, int);
  launcher_t launcher = (launcher_t)dlsym(h, "cerium_function_map_launcher");
  const char* types[4] = {"ntt", "int", "sud", "bco"};
  if (launcher)
    for (int k = 0; k < 2; k++)
      for (const char* t : types) std::printf("launcher %s %s %p\n", tags[k], t, launcher(t, k));
  return 0;
}
