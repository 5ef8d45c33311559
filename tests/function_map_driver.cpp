// Loads function_map_<p>.so plugins the way the reference runtime does (dlopen, dlsym of the two
// asm-labelled getters, call; cerium/runtime/execution/function.cpp:144-177) - all of them into this one
// process, as the runtime loads every partition of a function - and prints the maps they return, one
// "<plugin index> <stream|graph> <id> <launcher address>" line per entry.
//   driver [--preload <libcerium_b200.so>] <plugin> [<plugin> ...]
// --preload opens the library under its real name first, as a host program that binds a context does.
// TEST INFRASTRUCTURE: built by tests/test_function_map.py with g++; needs no GPU (the getters only
// build the maps).
#include <dlfcn.h>

#include <cstdint>
#include <cstdio>
#include <cstring>
#include <exception>
#include <unordered_map>

typedef std::unordered_map<uint32_t, void*> FunctionMapType;
typedef const FunctionMapType& (*map_function_t)();

int main(int argc, char** argv) {
  int first = 1;
  void* lib = nullptr;
  if (argc >= 3 && std::strcmp(argv[1], "--preload") == 0) {
    lib = dlopen(argv[2], RTLD_NOW | RTLD_GLOBAL);
    if (!lib) {
      std::fprintf(stderr, "dlopen: %s\n", dlerror());
      return 3;
    }
    first = 3;
  }
  if (argc <= first) return 2;
  const char* names[2] = {"__GET_FUNCTION_MAP__", "__GET_FUNCTION_MAP_CUGRAPH__"};
  const char* tags[2] = {"stream", "graph"};
  for (int a = first; a < argc; a++) {
    void* h = dlopen(argv[a], RTLD_LAZY);
    if (!h) {
      std::fprintf(stderr, "dlopen: %s\n", dlerror());
      return 3;
    }
    for (int k = 0; k < 2; k++) {
      map_function_t get = (map_function_t)dlsym(h, names[k]);
      if (!get) {
        std::fprintf(stderr, "dlsym %s: %s\n", names[k], dlerror());
        return 4;
      }
      try {
        const FunctionMapType& m = get();
        for (const auto& kv : m) std::printf("%d %s %u %p\n", a - first, tags[k], kv.first, kv.second);
      } catch (const std::exception& e) {
        std::printf("error %d %s\n", a - first, e.what());
      }
    }
    if (a == first) {
      typedef void* (*launcher_t)(const char*, int);
      // the launchers live in the library the plugin links, visible through the plugin's dependency chain
      launcher_t launcher = (launcher_t)dlsym(h, "cerium_function_map_launcher");
      const char* types[4] = {"ntt", "int", "sud", "bco"};
      if (launcher)
        for (int k = 0; k < 2; k++)
          for (const char* t : types) std::printf("launcher %s %s %p\n", tags[k], t, launcher(t, k));
    }
  }
  return 0;
}
