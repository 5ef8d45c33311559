// Executor of a compiled Cerium function: reads the compiler's kernel stream (the `ll.functions` /
// `functions<p>` records written by FusedKernel::write_instruction,
// cerium/compiler/backend/cuda_kernel.cc:1707-1916), builds the argument tables of every record once
// and replays the records in order on a CUDA stream, calling the launchers of the function's kernel
// plugin by kernel id - the stream mode of the reference runtime:
//   record parser                 FunctionMetaData          cerium/runtime/execution/function.h:269-347
//   term resolution               get_pointer_from_term     cerium/runtime/execution/function.cpp:464-503
//   base-conversion units         DeviceBaseConverter       cerium/runtime/execution/evaluator.cpp:1483-1608
//   SuD / PMU factors             compute_{sud,pmu}_factors cerium/runtime/execution/function.cpp:685-755
//   argument tables per record    make_program's build loop cerium/runtime/execution/function_execution.cpp:124-360
//   replay                        run_program_multithread_threadfn  function_execution.cpp:437-611
// With the plugin shim of this library installed as function_map_<p>.so the ntt / int / sud / bco
// records run on this library's kernels and the generic / pmu records on the launchers the compiler
// generated for the program (kept as function_map_<p>.orig.so): a compiled program runs unchanged.
// One process drives one partition (the reference runs one host thread per partition).
//
// Differences from the reference: records are addressed by field name, not by line number; register
// file and base-conversion buffers are sized from what the records use; mov records (no-ops in the
// reference's runtime too) are dropped; the modulus / Barrett / rotation tables the generated
// element-wise launchers expect are built here in the reference's layout (EvaluatorContext,
// evaluator.cpp:58-92, 233-260), since they are part of that launcher contract.  A drm record (the
// all-gather of limbs between partitions, Evaluator::drm, evaluator.cpp:1154-1251) runs on the
// communicator given at load: its sources are packed into this rank's block of a staging buffer,
// gathered in place, and unpacked to the record's destinations.  A call record loads the called function
// from the same program directory and binds its argument and result limbs to the caller's (the reference
// copies them in and out, function_execution.cpp:265-331, 508-600).  An rsv record (two-limb CRT composition) runs on the
// program's generated kernel with the factors of compute_rsv_factors.  ags / ard records (sums over the
// partitions: reduce-scatter / all-reduce, then reduction modulo each limb's prime) run on the communicator
// like drm.  Not served: remapable inputs - a function that holds one is refused at load.
#include <algorithm>
#include <cstring>
#include <fstream>
#include <map>
#include <sstream>
#include <stdexcept>
#include <unordered_map>

#include "internal.h"

#if !defined(CERIUM_EMU)
#include <dlfcn.h>
#endif

using namespace cerium;

namespace {

struct Term {
  enum Type { Reg, Bcu, Mem, Arg, Zero } type = Mem;
  std::string s;  // without the "[X]" (dead after this use) mark
};

struct Record {
  uint32_t id = 0;
  std::string type;
  std::vector<Term> outputs, inputs, scalars, remapables, comm_srcs, comm_dests;
  size_t comm_size = 0, comm_num_limbs = 0;
  std::string base_conv;
  std::vector<int32_t> rots;
  std::vector<uint32_t> sud, pmu, rsv, bases;
  std::string function_name;    // call records: the callee
  std::string function_args;    // call records: "<var:c0(limb)~caller term>, ..."
};

std::string strip(const std::string& v) {
  std::string o;
  for (char c : v)
    if (c != ' ' && c != '\t' && c != '\r' && c != '\n') o += c;
  return o;
}

std::vector<std::string> csv(const std::string& v) {
  std::vector<std::string> out;
  std::string cur;
  for (char c : strip(v)) {
    if (c == ',') {
      if (!cur.empty()) out.push_back(cur);
      cur.clear();
    } else {
      cur += c;
    }
  }
  if (!cur.empty()) out.push_back(cur);
  return out;
}

Term make_term(std::string s) {
  Term t;
  const size_t dead = s.find("[X]");
  if (dead != std::string::npos) s.erase(dead);
  t.s = s;
  // the first character decides (function.cpp:236-255)
  switch (s.empty() ? ' ' : s[0]) {
    case 'b': t.type = Term::Bcu; break;
    case 'r': t.type = Term::Reg; break;
    case 'f': t.type = Term::Arg; break;
    case 'Z': t.type = Term::Zero; break;
    default: t.type = Term::Mem; break;
  }
  return t;
}

std::vector<Term> terms(const std::string& v) {
  std::vector<Term> out;
  for (const std::string& s : csv(v)) out.push_back(make_term(s));
  return out;
}

template <typename T>
std::vector<T> numbers(const std::string& v) {
  std::vector<T> out;
  for (const std::string& s : csv(v)) out.push_back((T)std::stol(s));
  return out;
}

// Records are '}'-delimited; every field is a ".name: value" line.
bool parse_records(const std::string& path, std::vector<Record>& out, std::string& err) {
  std::ifstream f(path);
  if (!f.is_open()) {
    err = "cannot open " + path;
    return false;
  }
  std::string text;
  while (std::getline(f, text, '}')) {
    std::istringstream lines(text);
    std::string line;
    Record r;
    bool any = false;
    std::map<std::string, std::string> field;
    while (std::getline(lines, line)) {
      const size_t a = line.find_first_not_of(" \t");
      if (a == std::string::npos || line[a] != '.') continue;
      const size_t colon = line.find(':', a);
      if (colon == std::string::npos) continue;
      field[line.substr(a + 1, colon - a - 1)] = line.substr(colon + 1);
      any = true;
    }
    if (!any) continue;
    try {
      if (!field.count("id") || !field.count("type")) throw std::runtime_error("record without .id / .type");
      r.id = (uint32_t)std::stoul(strip(field["id"]));
      r.type = strip(field["type"]);
      r.outputs = terms(field["outputs"]);
      r.inputs = terms(field["inputs"]);
      r.scalars = terms(field["scalars"]);
      r.remapables = terms(field["reamapables"]);  // sic: the producer's spelling
      r.base_conv = field["base_conv"];
      r.rots = numbers<int32_t>(field["rots"]);
      r.sud = numbers<uint32_t>(field["sud"]);
      r.pmu = numbers<uint32_t>(field["pmu"]);
      r.rsv = numbers<uint32_t>(field["rsv"]);
      r.bases = numbers<uint32_t>(field["bases"]);
      r.comm_srcs = terms(field["comm_srcs"]);
      r.comm_dests = terms(field["comm_dests"]);
      r.function_name = strip(field["function_name"]);
      r.function_args = strip(field["function_args"]);
      if (!strip(field["comm_size"]).empty()) r.comm_size = std::stoul(strip(field["comm_size"]));
      if (!strip(field["comm_num_limbs"]).empty()) r.comm_num_limbs = std::stoul(strip(field["comm_num_limbs"]));
    } catch (const std::exception& e) {
      err = "bad record in " + path + ": " + e.what();
      return false;
    }
    out.push_back(std::move(r));
  }
  return true;
}

// "<b0: 0, 1, : 52, 53, ><b1: ...>" -> per unit: index, first list, second list
struct BcuSpec {
  int unit;
  std::vector<uint32_t> first, second;
};
std::vector<BcuSpec> parse_base_conv(const std::string& v) {
  std::vector<BcuSpec> out;
  std::string s = strip(v);
  size_t pos = 0;
  while ((pos = s.find('<', pos)) != std::string::npos) {
    const size_t end = s.find('>', pos);
    if (end == std::string::npos) break;
    std::string body = s.substr(pos + 1, end - pos - 1);
    pos = end + 1;
    if (body.size() < 2 || body[0] != 'b') continue;
    std::vector<std::string> parts;
    size_t a = 0, c;
    while ((c = body.find(':', a)) != std::string::npos) {
      parts.push_back(body.substr(a, c - a));
      a = c + 1;
    }
    parts.push_back(body.substr(a));
    BcuSpec b;
    b.unit = std::stoi(parts[0].substr(1));
    if (parts.size() > 1) b.first = numbers<uint32_t>(parts[1]);
    if (parts.size() > 2) b.second = numbers<uint32_t>(parts[2]);
    out.push_back(b);
  }
  return out;
}

// "<value:c0(3)~i1(3)>, <doubled:c1(0)~v4(0)>" -> (callee object "value:c0", limb 3, caller term "i1(3)")
struct CallArg {
  std::string object;
  uint32_t limb;
  std::string caller_term;
};
std::vector<CallArg> parse_call_args(const std::string& v) {
  std::vector<CallArg> out;
  const std::string s = strip(v);
  size_t pos = 0;
  while ((pos = s.find('<', pos)) != std::string::npos) {
    const size_t end = s.find('>', pos);
    if (end == std::string::npos) break;
    const std::string body = s.substr(pos + 1, end - pos - 1);
    pos = end + 1;
    const size_t tilde = body.find('~'), l = body.find('('), r = body.find(')');
    if (tilde == std::string::npos || l == std::string::npos || r == std::string::npos || l > tilde || r > tilde)
      throw std::runtime_error("bad call argument <" + body + ">");
    out.push_back({body.substr(0, l), (uint32_t)std::stoul(body.substr(l + 1, r - l - 1)), body.substr(tilde + 1)});
  }
  return out;
}

// The "Function Input Stream" / "Function Output Stream" lines of a callee's inputs<p> file
// ("f1 | value:c0 | [0,1,...]"): object -> the callee's own term for it.
bool parse_function_streams(const std::string& path, std::map<std::string, std::string>& object_to_term,
                            std::map<std::string, bool>& is_output, std::string& err) {
  std::ifstream f(path);
  if (!f.is_open()) {
    err = "cannot open " + path;
    return false;
  }
  std::string line;
  bool inside = false, output = false;
  while (std::getline(f, line)) {
    const std::string t = strip(line);
    if (t.empty()) continue;
    if (t.size() > 7 && t.compare(t.size() - 7, 7, "Stream:") == 0) {
      inside = t.compare(0, 8, "Function") == 0;
      output = t.find("Output") != std::string::npos;
      continue;
    }
    if (t == ";") {
      inside = false;
      continue;
    }
    if (!inside) continue;
    const size_t a = t.find('|'), b = t.find('|', a + 1);
    if (a == std::string::npos || b == std::string::npos) continue;
    object_to_term[t.substr(a + 1, b - a - 1)] = t.substr(0, a);
    is_output[t.substr(a + 1, b - a - 1)] = output;
  }
  return true;
}

}  // namespace

#if !defined(CERIUM_EMU)

namespace {

using W = uint32_t;  // the reference's limb word; compiled programs exist for 32-bit contexts only
using FunctionMapType = std::unordered_map<uint32_t, void*>;

// launcher signatures of the plugin contract (cerium/runtime/execution/device_utils.cu:33-77)
typedef void (*ewi_fn)(cudaStream_t&, W**, const W**, const W*, const W**, const size_t*, const uint32_t*, const W*,
                       const W*, const uint32_t*, const uint32_t**);
typedef void (*ntt_fn)(cudaStream_t&, W**, const W**, const uint32_t*, const size_t, const W*, const uint2*);
typedef void (*sud_fn)(cudaStream_t&, W**, const W**, const uint32_t*, const size_t, const W*, const uint2*, const W*,
                       const W*, const uint32_t*);
typedef void (*rsv_fn)(cudaStream_t&, W**, const W**, const W*, const W*, const W*, const uint32_t);
typedef void (*bco_fn)(cudaStream_t&, W**, const size_t*, const W**, const size_t*, const W**, const W**, const W**,
                       const W**, const size_t, const size_t);

// Pack / unpack of the exchange records (the reference's _copy_to_nccl_buffer_ / _copy_from_nccl_buffer_with_mod_,
// cerium/runtime/execution/device_utils.cu:290-340): limbs named by a pointer table <-> one contiguous staging
// buffer, 16 bytes per thread.  A null source packs zeros, a null destination is skipped; `bases` != null reduces
// every word modulo its limb's prime (sums of up to 16 residues below 2^28 arrive unreduced).
constexpr int kPackThreads = 256;
__global__ void __launch_bounds__(kPackThreads) pack_limbs_kernel(W* __restrict__ staging, const W* const* __restrict__ ins) {
  const W* src = ins[blockIdx.y];
  const size_t i = ((size_t)blockIdx.x * kPackThreads + threadIdx.x) * 4;
  uint4 v = make_uint4(0, 0, 0, 0);
  if (src != nullptr) v = *reinterpret_cast<const uint4*>(src + i);
  *reinterpret_cast<uint4*>(staging + (size_t)blockIdx.y * kN + i) = v;
}
__global__ void __launch_bounds__(kPackThreads)
    unpack_limbs_kernel(W* const* __restrict__ outs, const W* __restrict__ staging, const uint32_t* __restrict__ bases,
                        const W* __restrict__ moduli) {
  W* dst = outs[blockIdx.y];
  if (dst == nullptr) return;
  const size_t i = ((size_t)blockIdx.x * kPackThreads + threadIdx.x) * 4;
  uint4 v = *reinterpret_cast<const uint4*>(staging + (size_t)blockIdx.y * kN + i);
  if (bases != nullptr) {
    const W q = moduli[bases[blockIdx.y]];
    v.x %= q;
    v.y %= q;
    v.z %= q;
    v.w %= q;
  }
  *reinterpret_cast<uint4*>(dst + i) = v;
}

struct Unit {  // one base-conversion unit: input block, output block, the bases they hold right now
  std::vector<uint32_t> in_ids, out_ids;
  W* in_buf = nullptr;
  W* out_buf = nullptr;
};
constexpr int kUnitMaxIn = 48, kUnitMaxOut = 64;  // DeviceBaseConverter's block sizes (evaluator.h:36-38)

struct Step {
  enum Kind { Ewi, Ntt, Int, Sud, Bco, Drm, Call, Rsv, Ags, Ard } kind;
  // exchange records: device pointer tables of the limbs to pack and to unpack, prime index per unpacked limb
  const W* const* pack_tab = nullptr;
  W* const* unpack_tab = nullptr;
  const uint32_t* unpack_bases = nullptr;
  size_t n_pack = 0, n_unpack = 0;
  // rsv: CRT factors, the modulus product, its Barrett ratio (all as words) and the Barrett shift
  const W *rsv_factors = nullptr, *rsv_modulus = nullptr, *rsv_ratio = nullptr;
  uint32_t rsv_k = 0;
  cerium_comm* comm = nullptr;       // exchange records: the group of partitions the record spans
  cerium_program* callee = nullptr;  // call: the called function, its argument terms bound to this function's memory
  std::vector<std::pair<W*, const W*>> copy_back;  // call: results whose destination is also an argument (dst, src)
  // drm: host lists of the limbs to pack (this rank's sources) and to unpack (every rank's block)
  std::vector<const W*> pack;
  std::vector<W*> unpack;
  W* staging = nullptr;
  size_t comm_limbs = 0;
  void* fn = nullptr;
  uint32_t id = 0;
  // device tables (owned by the program's arena)
  W** outs = nullptr;
  const W** ins = nullptr;
  const W* scalars = nullptr;
  const uint32_t* bases = nullptr;
  size_t n_bases = 0;
  const uint32_t** rotmaps = nullptr;
  const W* sud_factors = nullptr;
  // bco
  const size_t *n_out = nullptr, *n_in = nullptr;
  const W** factors = nullptr;
  const W** out_moduli = nullptr;
  const W** ratios = nullptr;
  const W** ks = nullptr;
  size_t smem = 0, count = 0;
};

}  // namespace

struct cerium_program {
  cerium_context* ctx = nullptr;
  cerium_comm* comm = nullptr;
  void* plugin = nullptr;
  std::vector<Step> steps;
  std::vector<void*> allocs;                          // everything cudaMalloc'ed for this program
  W* regs = nullptr;
  std::map<std::string, W*> memory;                    // named program memory, one limb per term
  std::map<int, Unit> units;
  std::map<uint32_t, const uint32_t*> rot_tables;      // Galois element -> device inverse table
  const W *d_moduli = nullptr, *d_ratios = nullptr;
  const uint32_t* d_k = nullptr;
  cudaGraphExec_t graph = nullptr;                    // one captured run (cerium_program_capture), replayed by run
  std::vector<cerium_program*> callees;               // functions this one calls (owned)
  std::string functions_path;                          // <programs>/<function>/functions<p>
  int depth = 0;
};

namespace {
constexpr int kMaxCallDepth = 16;
cerium_program* load_program(cerium_context* ctx, const std::string& functions_path, const std::string& plugin_path,
                             const std::map<std::string, uint64_t>& scalars, cerium_comm* comm,
                             const std::map<std::string, W*>& bound, int depth);
}

namespace {

struct Loader {
  cerium_program* p;
  cerium_context* ctx;
  std::string err;

  void* dev_alloc(size_t bytes) {
    void* d = nullptr;
    if (cudaMalloc(&d, bytes ? bytes : 16) != cudaSuccess) throw std::runtime_error("cudaMalloc failed");
    p->allocs.push_back(d);
    return d;
  }
  template <typename T>
  T* upload(const std::vector<T>& v) {
    T* d = static_cast<T*>(dev_alloc(v.size() * sizeof(T)));
    if (!v.empty() && cudaMemcpy(d, v.data(), v.size() * sizeof(T), cudaMemcpyHostToDevice) != cudaSuccess)
      throw std::runtime_error("cudaMemcpy failed");
    return d;
  }
  W* limb_alloc(size_t limbs) {
    W* d = static_cast<W*>(dev_alloc(limbs * kN * sizeof(W)));
    if (cudaMemset(d, 0, limbs * kN * sizeof(W)) != cudaSuccess) throw std::runtime_error("cudaMemset failed");
    return d;
  }

  Unit& unit(int k) {
    auto it = p->units.find(k);
    if (it != p->units.end()) return it->second;
    Unit u;
    u.in_buf = limb_alloc(kUnitMaxIn);
    u.out_buf = limb_alloc(kUnitMaxOut);
    return p->units.emplace(k, u).first->second;
  }

  // DeviceBaseConverter::get_pointer: the inputs first, then the outputs
  W* unit_pointer(int k, uint32_t base) {
    Unit& u = unit(k);
    for (size_t i = 0; i < u.in_ids.size(); i++)
      if (u.in_ids[i] == base) return u.in_buf + i * kN;
    for (size_t i = 0; i < u.out_ids.size(); i++)
      if (u.out_ids[i] == base) return u.out_buf + i * kN;
    throw std::runtime_error("base-conversion unit b" + std::to_string(k) + " holds no limb of prime " + std::to_string(base));
  }

  W* pointer(const Term& t) {
    switch (t.type) {
      case Term::Zero: return nullptr;
      case Term::Reg: return p->regs + (size_t)std::stoul(t.s.substr(1)) * kN;
      case Term::Bcu: {
        const size_t l = t.s.find('('), r = t.s.find(')');
        if (l == std::string::npos || r == std::string::npos) throw std::runtime_error("bad unit term " + t.s);
        return unit_pointer(std::stoi(t.s.substr(1, l - 1)), (uint32_t)std::stoul(t.s.substr(l + 1, r - l - 1)));
      }
      default: {  // named program memory (and function arguments, which a single function treats alike)
        auto it = p->memory.find(t.s);
        if (it != p->memory.end()) return it->second;
        W* d = limb_alloc(1);
        p->memory[t.s] = d;
        return d;
      }
    }
  }

  std::vector<W*> pointers(const std::vector<Term>& ts) {
    std::vector<W*> v;
    for (const Term& t : ts) v.push_back(pointer(t));
    return v;
  }

  uint64_t product_mod(const std::vector<uint32_t>& ids, uint64_t q) {
    uint64_t r = 1 % q;
    for (uint32_t i : ids) {
      if (i >= (uint32_t)ctx->n_primes) throw std::runtime_error("prime index out of range in a factor list");
      r = host::mulmod(r, ctx->moduli[i] % q, q);
    }
    return r;
  }

  const uint32_t* rotation_table(int32_t step) {
    const uint32_t elt = cerium_galois_elt_from_step(step, kLogN);
    if (elt == 0) throw std::runtime_error("rotation step out of range");
    auto it = p->rot_tables.find(elt);
    if (it != p->rot_tables.end()) return it->second;
    // generate_table_ntt, then its inverse: inv[table[i]] = i (cerium/runtime/math/galois.cpp:30-77;
    // the generated kernels scatter through it, evaluator.cpp:241-249)
    std::vector<uint32_t> inv(kN);
    auto brev = [](uint32_t x, int bits) {
      uint32_t r = 0;
      for (int b = 0; b < bits; b++) r |= ((x >> b) & 1u) << (bits - 1 - b);
      return r;
    };
    for (uint32_t i = 0; i < (uint32_t)kN; i++) {
      const uint32_t reversed = brev(i + (uint32_t)kN, kLogN + 1);
      const uint64_t raw = (((uint64_t)elt * reversed) >> 1) & (uint64_t)(kN - 1);
      inv[brev((uint32_t)raw, kLogN)] = i;
    }
    const uint32_t* d = upload(inv);
    p->rot_tables[elt] = d;
    return d;
  }

  void reference_tables() {
    // EvaluatorContext::init_params: modulus, floor(2^58 / q), 58 per prime
    std::vector<W> mod, ratio;
    std::vector<uint32_t> k;
    for (int i = 0; i < ctx->n_primes; i++) {
      mod.push_back((W)ctx->moduli[i]);
      ratio.push_back((W)(((uint64_t)1 << 58) / ctx->moduli[i]));
      k.push_back(58);
    }
    p->d_moduli = upload(mod);
    p->d_ratios = upload(ratio);
    p->d_k = upload(k);
  }

  // The communicator an exchange record runs on: all partitions, or the group of .comm_size consecutive
  // partitions that holds this one (cerium/runtime/cuda/nccl_ops.cu:185-215).
  cerium_comm* group(const Record& r, const char* what) {
    cerium_comm* c = nullptr;
    if (r.comm_size == 0 || comm_subgroup(p->comm, (int)r.comm_size, &c) != CERIUM_OK)
      throw std::runtime_error(std::string(what) + " record " + std::to_string(r.id) + " spans " + std::to_string(r.comm_size) +
                               " partitions: " + cerium_last_error());
    return c;
  }

  void build(const std::vector<Record>& recs, const FunctionMapType& fmap,
             const std::map<std::string, uint64_t>& scalar_values) {
    // register file: as many registers as the records name
    size_t max_reg = 0;
    bool any_reg = false;
    for (const Record& r : recs)
      for (const auto* list : {&r.outputs, &r.inputs})
        for (const Term& t : *list)
          if (t.type == Term::Reg) {
            max_reg = std::max(max_reg, (size_t)std::stoul(t.s.substr(1)));
            any_reg = true;
          }
    if (any_reg) p->regs = limb_alloc(max_reg + 1);
    reference_tables();
    // sub-group communicators are created collectively: every partition asks for them in the same order
    if (p->comm != nullptr) {
      std::vector<int> sizes;
      for (const Record& r : recs)
        if ((r.type == "drm" || r.type == "ags" || r.type == "ard") && r.comm_size > 0 && (int)r.comm_size != p->comm->world &&
            std::find(sizes.begin(), sizes.end(), (int)r.comm_size) == sizes.end())
          sizes.push_back((int)r.comm_size);
      std::sort(sizes.rbegin(), sizes.rend());
      for (int sz : sizes) {
        cerium_comm* c = nullptr;
        if (comm_subgroup(p->comm, sz, &c) != CERIUM_OK) throw std::runtime_error(cerium_last_error());
      }
    }
    for (const Record& r : recs) {
      const std::string& ty = r.type;
      if (ty == "mov") continue;  // outputs alias inputs: nothing to run (the reference skips them too)
      if (ty == "ags" || ty == "ard") {
        // Evaluator::ags / ard (evaluator.cpp:1253-1481): the `gather` list (.comm_dests; world x limbs for ags,
        // limbs for ard; Z = a zero limb) is packed into a staging buffer, summed over the partitions - ags:
        // reduce-scatter, this partition keeps block `rank`; ard: all-reduce - and the `scatter` list
        // (.comm_srcs) receives the sums reduced modulo the primes of .bases.
        cerium_comm* comm = p->comm;
        if (comm == nullptr) throw std::runtime_error("record " + std::to_string(r.id) + " is an " + ty + " record: the function needs a communicator");
        comm = group(r, ty.c_str());
        const size_t blocks = ty == "ags" ? r.comm_size : 1;
        if (r.comm_dests.size() > blocks * r.comm_num_limbs || r.comm_srcs.size() > r.comm_num_limbs || r.bases.size() < r.comm_srcs.size())
          throw std::runtime_error(ty + " record " + std::to_string(r.id) + " lists more limbs than it exchanges");
        for (uint32_t b : r.bases)
          if (b >= (uint32_t)ctx->n_primes) throw std::runtime_error("prime index out of range in .bases");
        Step s{};
        s.kind = ty == "ags" ? Step::Ags : Step::Ard;
        s.comm = comm;
        s.id = r.id;
        s.comm_limbs = r.comm_num_limbs;
        // zero-filled: limbs past the gather list stay zero; ags receives into a block of its own behind them
        s.staging = limb_alloc((blocks + (ty == "ags" ? 1 : 0)) * r.comm_num_limbs);
        std::vector<const W*> gather;
        for (const Term& t : r.comm_dests) gather.push_back(pointer(t));
        std::vector<W*> scatter = pointers(r.comm_srcs);
        s.pack_tab = upload(gather);
        s.unpack_tab = upload(scatter);
        s.unpack_bases = upload(r.bases);
        s.n_pack = gather.size();
        s.n_unpack = scatter.size();
        p->steps.push_back(s);
        continue;
      }
      if (ty == "call") {
        // The call case of CeriumFunction::make_program / run (function_execution.cpp:265-331, 508-600): the callee
        // is the function `function_name` of the same program directory; .function_args pairs its argument and
        // result limbs with THIS function's terms.  The reference copies arguments in and results out around
        // the callee's run; here the callee's terms are bound to the caller's limbs (no copies), except a
        // result whose destination is also an argument, which keeps the copy.
        if (r.function_name.empty()) throw std::runtime_error("call record " + std::to_string(r.id) + " names no function");
        if (p->depth + 1 > kMaxCallDepth) throw std::runtime_error("calls nest deeper than " + std::to_string(kMaxCallDepth));
        const size_t slash = p->functions_path.find_last_of('/');
        const std::string file = slash == std::string::npos ? p->functions_path : p->functions_path.substr(slash + 1);
        const std::string fdir = slash == std::string::npos ? std::string(".") : p->functions_path.substr(0, slash);
        const size_t up = fdir.find_last_of('/');
        const std::string base = up == std::string::npos ? std::string(".") : fdir.substr(0, up);
        if (file.compare(0, 9, "functions") != 0) throw std::runtime_error("a function that calls another must be loaded from <programs>/<function>/functions<p>");
        const std::string part = file.substr(9);
        const std::string cdir = base + "/" + r.function_name;
        std::map<std::string, std::string> object_to_term;
        std::map<std::string, bool> is_output;
        std::string perr;
        if (!parse_function_streams(cdir + "/inputs" + part, object_to_term, is_output, perr))
          throw std::runtime_error("call record " + std::to_string(r.id) + ": " + perr);
        const std::vector<CallArg> args = parse_call_args(r.function_args);
        std::map<std::string, W*> bound;
        std::vector<W*> arg_ptrs;
        std::vector<std::pair<std::string, W*>> late;  // results that must be copied after the run
        for (int pass = 0; pass < 2; pass++)           // arguments first, so that results can be checked against them
          for (const CallArg& a : args) {
            auto ot = object_to_term.find(a.object);
            if (ot == object_to_term.end()) throw std::runtime_error("function " + r.function_name + " has no argument or result '" + a.object + "'");
            if (is_output[a.object] != (pass == 1)) continue;
            const std::string term = ot->second + "(" + std::to_string(a.limb) + ")";
            W* here = pointer(make_term(a.caller_term));
            if (pass == 0) {
              bound[term] = here;
              arg_ptrs.push_back(here);
            } else if (std::find(arg_ptrs.begin(), arg_ptrs.end(), here) != arg_ptrs.end()) {
              late.push_back({term, here});
            } else {
              bound[term] = here;
            }
          }
        cerium_program* callee = load_program(ctx, cdir + "/functions" + part, cdir + "/function_map_" + part + ".so",
                                              scalar_values, p->comm, bound, p->depth + 1);
        p->callees.push_back(callee);
        Step s{};
        s.kind = Step::Call;
        s.id = r.id;
        s.callee = callee;
        for (const auto& l : late) {
          auto m = callee->memory.find(l.first);
          if (m != callee->memory.end()) s.copy_back.push_back({l.second, m->second});
        }
        p->steps.push_back(s);
        continue;
      }
      const std::vector<BcuSpec> specs = parse_base_conv(r.base_conv);
      // unit state changes happen BEFORE the record's terms are resolved (parse_term_base_conv_vec)
      if (ty == "generic" || ty == "int" || ty == "drm")
        for (const BcuSpec& b : specs) {
          Unit& u = unit(b.unit);
          u.in_ids.insert(u.in_ids.end(), b.first.begin(), b.first.end());
          if (u.in_ids.size() > (size_t)kUnitMaxIn) throw std::runtime_error("base-conversion unit overflows its input block");
        }
      if (ty == "bco")
        for (const BcuSpec& b : specs) {
          Unit& u = unit(b.unit);
          u.out_ids = b.second;
          if (u.out_ids.size() > (size_t)kUnitMaxOut) throw std::runtime_error("base-conversion unit overflows its output block");
        }
      if (ty == "drm") {
        cerium_comm* comm = p->comm;
        if (comm == nullptr) throw std::runtime_error("record " + std::to_string(r.id) + " is a drm (all-gather) record: the function needs a communicator");
        comm = group(r, "drm");
        if (r.comm_srcs.size() > r.comm_num_limbs || r.comm_dests.size() > r.comm_size * r.comm_num_limbs)
          throw std::runtime_error("drm record " + std::to_string(r.id) + " lists more limbs than it exchanges");
        Step s{};
        s.kind = Step::Drm;
        s.comm = comm;
        s.id = r.id;
        s.comm_limbs = r.comm_num_limbs;
        s.staging = limb_alloc(r.comm_size * r.comm_num_limbs);
        for (const Term& t : r.comm_srcs) s.pack.push_back(pointer(t));      // null = a zero limb
        for (const Term& t : r.comm_dests) s.unpack.push_back(pointer(t));   // null = not wanted here
        s.pack_tab = upload(s.pack);
        s.unpack_tab = upload(s.unpack);
        s.n_pack = s.pack.size();
        s.n_unpack = s.unpack.size();
        p->steps.push_back(s);
        continue;
      }
      auto it = fmap.find(r.id);
      if (it == fmap.end() || it->second == nullptr)
        throw std::runtime_error("the plugin has no launcher for record " + std::to_string(r.id) + " (" + ty + ")");
      Step s{};
      s.fn = it->second;
      s.id = r.id;
      if (ty == "bco") {
        if (specs.empty()) continue;
        std::vector<W*> outs;
        std::vector<const W*> ins, facs, omods, ratios, ks;
        std::vector<size_t> n_out, n_in;
        size_t smem_words = 0;
        for (const BcuSpec& b : specs) {
          Unit& u = unit(b.unit);
          if (u.in_ids != b.first) throw std::runtime_error("base-conversion unit b" + std::to_string(b.unit) + " does not hold the inputs record " + std::to_string(r.id) + " converts");
          const size_t I = u.in_ids.size(), O = u.out_ids.size();
          if (I == 0 || O == 0) throw std::runtime_error("empty base conversion");
          // F[j][i] = [Qhat_i^-1]_{q_i} * (Qhat_i mod p_j) mod p_j  (DeviceBaseConverter::set_output_bases)
          std::vector<uint64_t> inv(I);
          for (size_t i = 0; i < I; i++) {
            const uint64_t qi = ctx->moduli[u.in_ids[i]];
            uint64_t prod = 1 % qi;
            for (size_t k = 0; k < I; k++)
              if (k != i) prod = host::mulmod(prod, ctx->moduli[u.in_ids[k]] % qi, qi);
            inv[i] = I > 1 ? host::invmod(prod, qi) : 1;
          }
          std::vector<W> F(O * I), om(O), ra(O);
          std::vector<uint32_t> kk(O, 58);
          for (size_t j = 0; j < O; j++) {
            if (u.out_ids[j] >= (uint32_t)ctx->n_primes) throw std::runtime_error("prime index out of range");
            const uint64_t pj = ctx->moduli[u.out_ids[j]];
            om[j] = (W)pj;
            ra[j] = (W)(((uint64_t)1 << 58) / pj);
            for (size_t i = 0; i < I; i++) {
              uint64_t qhat = 1 % pj;
              for (size_t k = 0; k < I; k++)
                if (k != i) qhat = host::mulmod(qhat, ctx->moduli[u.in_ids[k]] % pj, pj);
              F[j * I + i] = (W)host::mulmod(inv[i] % pj, qhat, pj);
            }
          }
          outs.push_back(u.out_buf);
          ins.push_back(u.in_buf);
          n_out.push_back(O);
          n_in.push_back(I);
          facs.push_back(upload(F));
          omods.push_back(upload(om));
          ratios.push_back(upload(ra));
          ks.push_back(reinterpret_cast<const W*>(upload(kk)));
          // Evaluator::fn_bco's shared-memory size
          smem_words = std::max(smem_words, (O * I / 32 + 1) * 32 + I * 256);
          u.in_ids.clear();  // set_input_bases({}) after the conversion is built (evaluator.cpp:939)
        }
        s.kind = Step::Bco;
        s.outs = upload(outs);
        s.ins = upload(ins);
        s.n_out = upload(n_out);
        s.n_in = upload(n_in);
        s.factors = upload(facs);
        s.out_moduli = upload(omods);
        s.ratios = upload(ratios);
        s.ks = upload(ks);
        s.smem = smem_words * sizeof(W);
        s.count = specs.size();
        p->steps.push_back(s);
        continue;
      }
      if (r.outputs.empty()) continue;
      if (!r.remapables.empty()) throw std::runtime_error("record " + std::to_string(r.id) + " reads remapable inputs, which this executor does not serve");
      std::vector<W*> ins_h = pointers(r.inputs);
      std::vector<W*> outs_h = pointers(r.outputs);
      std::vector<const W*> ins_c(ins_h.begin(), ins_h.end());
      s.outs = upload(outs_h);
      s.ins = upload(ins_c);
      for (uint32_t b : r.bases)
        if (b >= (uint32_t)ctx->n_primes) throw std::runtime_error("prime index out of range in .bases");
      s.bases = upload(r.bases);
      s.n_bases = r.bases.size();
      if (ty == "generic" || ty == "pmu") {
        s.kind = Step::Ewi;
        std::vector<W> sc;
        if (ty == "pmu") {
          // compute_pmu_factors: [prod pmu bases] mod q_i for every prime of the context
          for (int i = 0; i < ctx->n_primes; i++) sc.push_back((W)product_mod(r.pmu, ctx->moduli[i]));
        } else {
          for (const Term& t : r.scalars) {
            auto sv = scalar_values.find(t.s);
            if (sv == scalar_values.end()) throw std::runtime_error("no value given for scalar " + t.s);
            sc.push_back((W)sv->second);
          }
        }
        s.scalars = upload(sc);
        if (!r.rots.empty()) {
          std::vector<const uint32_t*> maps;
          for (int32_t amt : r.rots) maps.push_back(rotation_table(amt));
          s.rotmaps = upload(maps);
        }
      } else if (ty == "rsv") {
        // compute_rsv_factors (function_execution.cpp:53-99): for the primes of .rsv, factor_i =
        // (Q / q_i) * [(Q / q_i)^-1]_{q_i} as a multi-word integer (one 64-bit word per prime, stored as
        // 32-bit words), the product Q, and floor(2^k / Q) with k = floor(log2 Q) + 63.  The generated
        // kernel composes x = sum x_i * factor_i mod Q from them.  Two primes below 2^32: everything fits
        // in 64-bit words, which is the only shape the compiler emits (double rescale, ModRaise).
        s.kind = Step::Rsv;
        if (r.rsv.size() != 2) throw std::runtime_error("rsv record " + std::to_string(r.id) + " resolves " + std::to_string(r.rsv.size()) + " primes; two are served");
        for (uint32_t b : r.rsv)
          if (b >= (uint32_t)ctx->n_primes) throw std::runtime_error("prime index out of range in .rsv");
        const uint64_t q0 = ctx->moduli[r.rsv[0]], q1 = ctx->moduli[r.rsv[1]];
        if (q0 >> 32 || q1 >> 32) throw std::runtime_error("rsv primes must be below 2^32");
        const uint64_t Q = q0 * q1;
        const uint64_t f0 = q1 * host::invmod(q1 % q0, q0), f1 = q0 * host::invmod(q0 % q1, q1);
        std::vector<W> fac = {(W)f0, (W)(f0 >> 32), (W)f1, (W)(f1 >> 32)};
        std::vector<W> mod = {(W)Q, (W)(Q >> 32)};
        uint32_t log2q = 0;
        while ((Q >> (log2q + 1)) != 0) log2q++;
        const uint32_t k = log2q + 63;
        const unsigned __int128 ratio = ((unsigned __int128)1 << k) / Q;
        std::vector<W> rat = {(W)(uint64_t)ratio, (W)((uint64_t)ratio >> 32)};
        s.rsv_factors = upload(fac);
        s.rsv_modulus = upload(mod);
        s.rsv_ratio = upload(rat);
        s.rsv_k = k;
      } else if (ty == "ntt") {
        s.kind = Step::Ntt;
      } else if (ty == "int") {
        s.kind = Step::Int;
      } else if (ty == "sud") {
        s.kind = Step::Sud;
        // compute_sud_factors: [(prod divide bases)^-1] mod q_i for every prime (0 where not invertible)
        std::vector<W> fac;
        for (int i = 0; i < ctx->n_primes; i++) {
          const uint64_t q = ctx->moduli[i];
          fac.push_back((W)host::invmod(product_mod(r.sud, q), q));
        }
        s.sud_factors = upload(fac);
      } else {
        throw std::runtime_error("unknown record type '" + ty + "'");
      }
      p->steps.push_back(s);
    }
  }
};

cerium_program* load_program(cerium_context* ctx, const std::string& functions_path, const std::string& plugin_path,
                             const std::map<std::string, uint64_t>& scalars, cerium_comm* comm,
                             const std::map<std::string, W*>& bound, int depth) {
  std::vector<Record> recs;
  std::string err;
  if (!parse_records(functions_path, recs, err)) throw std::runtime_error(err);
  void* h = dlopen(plugin_path.c_str(), RTLD_LAZY | RTLD_LOCAL);
  if (!h) throw std::runtime_error(std::string("cannot load the plugin: ") + dlerror());
  typedef const FunctionMapType& (*getter_t)();
  getter_t getter = (getter_t)dlsym(h, "__GET_FUNCTION_MAP__");
  if (!getter) {
    dlclose(h);
    throw std::runtime_error("the plugin " + plugin_path + " does not export __GET_FUNCTION_MAP__");
  }
  auto* p = new cerium_program();
  p->ctx = ctx;
  p->comm = comm;
  p->plugin = h;
  p->functions_path = functions_path;
  p->depth = depth;
  p->memory = bound;  // a called function's argument and result limbs live in its caller
  try {
    const FunctionMapType& fmap = getter();
    Loader ld{p, ctx, {}};
    ld.build(recs, fmap, scalars);
  } catch (...) {
    cerium_program_destroy(p);
    throw;
  }
  return p;
}

}  // namespace

extern "C" {

int cerium_program_load(cerium_context* ctx, cerium_program** out, const char* functions_path, const char* plugin_path,
                        const char* const* scalar_terms, const uint64_t* scalar_values, int n_scalars, cerium_comm* comm) {
  if (!ctx || !out || !functions_path || !plugin_path) return fail(CERIUM_ERR_INVALID, "program_load: null argument");
  if (n_scalars < 0 || (n_scalars > 0 && (!scalar_terms || !scalar_values))) return fail(CERIUM_ERR_INVALID, "program_load: bad scalar list");
  if (ctx->word_bits != 32)
    return fail(CERIUM_ERR_UNSUPPORTED, "program_load: compiled programs carry generated 32-bit kernels; the context must use 32-bit words");
  DeviceGuard guard(ctx->device);
  if (!guard.ok) return fail(CERIUM_ERR_CUDA, "program_load: cannot select device");
  std::map<std::string, uint64_t> scalars;
  for (int i = 0; i < n_scalars; i++) scalars[strip(scalar_terms[i])] = scalar_values[i];
  try {
    *out = load_program(ctx, functions_path, plugin_path, scalars, comm, {}, 0);
  } catch (const std::exception& e) {
    return fail(CERIUM_ERR_INVALID, std::string("program_load: ") + e.what());
  }
  return CERIUM_OK;
}

int cerium_program_destroy(cerium_program* p) {
  if (!p) return CERIUM_OK;
  DeviceGuard guard(p->ctx->device);
  for (cerium_program* c : p->callees) cerium_program_destroy(c);
  if (p->graph != nullptr) cudaGraphExecDestroy(p->graph);
  for (void* d : p->allocs) cudaFree(d);
  // the plugin stays loaded: its maps are referenced for the life of the process
  delete p;
  return CERIUM_OK;
}

int cerium_program_num_steps(const cerium_program* p) { return p ? (int)p->steps.size() : 0; }

int cerium_program_memory(cerium_program* p, const char* term, void** device_ptr) {
  if (!p || !term || !device_ptr) return fail(CERIUM_ERR_INVALID, "program_memory: null argument");
  auto it = p->memory.find(strip(term));
  if (it == p->memory.end()) return fail(CERIUM_ERR_INVALID, std::string("program_memory: the function names no memory term '") + term + "'");
  *device_ptr = it->second;
  return CERIUM_OK;
}

static int program_copy(cerium_program* p, const char* name, const uint32_t* limb_ids, int n_limbs, void* host,
                        void* stream, bool to_device) {
  const char* what = to_device ? "program_write" : "program_read";
  if (!p || !name || !limb_ids || !host || n_limbs < 0) return fail(CERIUM_ERR_INVALID, std::string(what) + ": null argument");
  DeviceGuard guard(p->ctx->device);
  if (!guard.ok) return fail(CERIUM_ERR_CUDA, std::string(what) + ": cannot select device");
  const size_t bytes = ((size_t)1 << p->ctx->logn) * sizeof(uint32_t);
  cudaStream_t st = (cudaStream_t)stream;
  for (int i = 0; i < n_limbs; ++i) {
    const std::string term = std::string(name) + "(" + std::to_string(limb_ids[i]) + ")";
    auto it = p->memory.find(term);
    if (it == p->memory.end()) return fail(CERIUM_ERR_INVALID, std::string(what) + ": the function names no memory term '" + term + "'");
    char* h = (char*)host + (size_t)i * bytes;
    cudaError_t e = to_device ? cudaMemcpyAsync(it->second, h, bytes, cudaMemcpyHostToDevice, st)
                              : cudaMemcpyAsync(h, it->second, bytes, cudaMemcpyDeviceToHost, st);
    if (e != cudaSuccess) return fail(CERIUM_ERR_CUDA, std::string(what) + ": " + cudaGetErrorString(e));
  }
  cudaError_t e = cudaStreamSynchronize(st);
  if (e != cudaSuccess) return fail(CERIUM_ERR_CUDA, std::string(what) + ": " + cudaGetErrorString(e));
  return CERIUM_OK;
}

int cerium_program_write(cerium_program* p, const char* name, const uint32_t* limb_ids, int n_limbs, const void* host,
                         void* stream) {
  return program_copy(p, name, limb_ids, n_limbs, const_cast<void*>(host), stream, true);
}

int cerium_program_read(cerium_program* p, const char* name, const uint32_t* limb_ids, int n_limbs, void* host, void* stream) {
  return program_copy(p, name, limb_ids, n_limbs, host, stream, false);
}

static int run_steps(cerium_program* p, cudaStream_t st) {
  try {
    for (const Step& s : p->steps) {
      switch (s.kind) {
        case Step::Ewi:
          ((ewi_fn)s.fn)(st, s.outs, s.ins, s.scalars, nullptr, nullptr, s.bases, p->d_moduli, p->d_ratios, p->d_k, s.rotmaps);
          break;
        case Step::Ntt:
        case Step::Int:
          // the reference's root tables are not rebuilt here: the transform records are expected to run on
          // this library's launchers, which use the bound context's tables
          ((ntt_fn)s.fn)(st, s.outs, s.ins, s.bases, s.n_bases, p->d_moduli, nullptr);
          break;
        case Step::Sud:
          ((sud_fn)s.fn)(st, s.outs, s.ins, s.bases, s.n_bases, p->d_moduli, nullptr, s.sud_factors, p->d_ratios, p->d_k);
          break;
        case Step::Bco:
          ((bco_fn)s.fn)(st, s.outs, s.n_out, s.ins, s.n_in, s.factors, s.out_moduli, s.ratios, s.ks, s.smem, s.count);
          break;
        case Step::Rsv:
          ((rsv_fn)s.fn)(st, s.outs, s.ins, s.rsv_factors, s.rsv_modulus, s.rsv_ratio, s.rsv_k);
          break;
        case Step::Call: {
          if (int rc = run_steps(s.callee, st)) return rc;
          for (const auto& c : s.copy_back)
            CERIUM_CUDA(cudaMemcpyAsync(c.first, c.second, (size_t)kN * sizeof(W), cudaMemcpyDeviceToDevice, st));
          break;
        }
        case Step::Drm: {
          const size_t limb = (size_t)kN * sizeof(W);
          W* mine = s.staging + (size_t)s.comm->rank * s.comm_limbs * kN;
          const dim3 grid(kN / (kPackThreads * 4));
          if (s.n_pack) pack_limbs_kernel<<<dim3(grid.x, (unsigned)s.n_pack), kPackThreads, 0, st>>>(mine, s.pack_tab);
          if (int rc = comm_allgather(s.comm, s.staging, mine, s.comm_limbs * limb, st)) return rc;
          if (s.n_unpack)
            unpack_limbs_kernel<<<dim3(grid.x, (unsigned)s.n_unpack), kPackThreads, 0, st>>>(s.unpack_tab, s.staging, nullptr, nullptr);
          break;
        }
        case Step::Ags:
        case Step::Ard: {
          const dim3 grid(kN / (kPackThreads * 4));
          if (s.n_pack) pack_limbs_kernel<<<dim3(grid.x, (unsigned)s.n_pack), kPackThreads, 0, st>>>(s.staging, s.pack_tab);
          const W* sums = s.staging;
          if (s.kind == Step::Ags) {
            W* mine = s.staging + (size_t)s.comm->world * s.comm_limbs * kN;
            if (int rc = comm_reducescatter_sum(s.comm, mine, s.staging, s.comm_limbs * kN, 32, st)) return rc;
            sums = mine;
          } else {
            if (int rc = comm_allreduce_sum(s.comm, s.staging, s.staging, s.comm_limbs * kN, 32, st)) return rc;
          }
          if (s.n_unpack)
            unpack_limbs_kernel<<<dim3(grid.x, (unsigned)s.n_unpack), kPackThreads, 0, st>>>(s.unpack_tab, sums, s.unpack_bases, p->d_moduli);
          break;
        }
      }
    }
  } catch (const std::exception& e) {
    return fail(CERIUM_ERR_CUDA, std::string("program_run: ") + e.what());
  }
  CERIUM_LAUNCH_CHECK("program_run");
  return CERIUM_OK;
}


int cerium_program_run(cerium_program* p, void* stream) {
  if (!p) return fail(CERIUM_ERR_INVALID, "program_run: null program");
  cerium_context* ctx = p->ctx;
  DeviceGuard guard(ctx->device);
  if (!guard.ok) return fail(CERIUM_ERR_CUDA, "program_run: cannot select device");
  if (p->graph != nullptr) {
    CERIUM_CUDA(cudaGraphLaunch(p->graph, (cudaStream_t)stream));
    return CERIUM_OK;
  }
  // the launchers of this library find their tables through the context bound to the device
  if (int rc = cerium_function_map_bind(ctx, ctx->device)) return fail(rc, "program_run: cannot bind the context");
  return run_steps(p, (cudaStream_t)stream);
}

// One run recorded into a CUDA graph on a stream of its own (every table a record's launcher takes was built
// at load and never changes, so the recording stays valid for the life of the program); exchange records
// are captured with it.  The reference builds its graph node by node (function_execution.cpp:670-1096).
int cerium_program_capture(cerium_program* p) {
  if (!p) return fail(CERIUM_ERR_INVALID, "program_capture: null program");
  if (p->graph != nullptr) return CERIUM_OK;
  cerium_context* ctx = p->ctx;
  DeviceGuard guard(ctx->device);
  if (!guard.ok) return fail(CERIUM_ERR_CUDA, "program_capture: cannot select device");
  if (int rc = cerium_function_map_bind(ctx, ctx->device)) return fail(rc, "program_capture: cannot bind the context");
  cudaStream_t st = nullptr;
  CERIUM_CUDA(cudaStreamCreateWithFlags(&st, cudaStreamNonBlocking));
  cudaGraph_t g = nullptr;
  cudaError_t e = cudaStreamBeginCapture(st, cudaStreamCaptureModeRelaxed);
  int rc = CERIUM_OK;
  if (e == cudaSuccess) {
    rc = run_steps(p, st);
    e = cudaStreamEndCapture(st, &g);   // always ended, also after a failed step, so that the stream leaves capture mode
  }
  cudaGraphExec_t exec = nullptr;
  if (rc == CERIUM_OK && e == cudaSuccess && g != nullptr) e = cudaGraphInstantiate(&exec, g, 0);
  if (g != nullptr) cudaGraphDestroy(g);
  cudaStreamDestroy(st);
  if (rc != CERIUM_OK) return rc;
  if (e != cudaSuccess || exec == nullptr) {
    cudaGetLastError();
    return fail(CERIUM_ERR_CUDA, std::string("program_capture: ") + cudaGetErrorString(e));
  }
  p->graph = exec;
  return CERIUM_OK;
}

}  // extern "C"

#else  // CERIUM_EMU: the executor drives a kernel plugin, which needs the CUDA runtime

struct cerium_program {};
extern "C" {
int cerium_program_load(cerium_context*, cerium_program**, const char*, const char*, const char* const*, const uint64_t*, int,
                        cerium_comm*) {
  return fail(CERIUM_ERR_UNSUPPORTED, "program_load: not part of the host-only test build");
}
int cerium_program_destroy(cerium_program*) { return CERIUM_OK; }
int cerium_program_num_steps(const cerium_program*) { return 0; }
int cerium_program_memory(cerium_program*, const char*, void**) { return CERIUM_ERR_UNSUPPORTED; }
int cerium_program_write(cerium_program*, const char*, const uint32_t*, int, const void*, void*) { return CERIUM_ERR_UNSUPPORTED; }
int cerium_program_read(cerium_program*, const char*, const uint32_t*, int, void*, void*) { return CERIUM_ERR_UNSUPPORTED; }
int cerium_program_run(cerium_program*, void*) { return CERIUM_ERR_UNSUPPORTED; }
int cerium_program_capture(cerium_program*) { return CERIUM_ERR_UNSUPPORTED; }
}

#endif  // !CERIUM_EMU

extern "C" int cerium_program_inspect(const char* functions_path, char* buf, size_t buf_bytes, int* n_records) {
  if (!functions_path || !n_records) return fail(CERIUM_ERR_INVALID, "program_inspect: null argument");
  std::vector<Record> recs;
  std::string err;
  if (!parse_records(functions_path, recs, err)) return fail(CERIUM_ERR_INVALID, "program_inspect: " + err);
  *n_records = (int)recs.size();
  std::ostringstream s;
  for (const Record& r : recs) {
    size_t call_args = 0;
    try {
      call_args = parse_call_args(r.function_args).size();
    } catch (const std::exception& e) {
      return fail(CERIUM_ERR_INVALID, std::string("program_inspect: ") + e.what());
    }
    s << r.id << ' ' << r.type << ' ' << r.outputs.size() << ' ' << r.inputs.size() << ' ' << r.bases.size() << ' '
      << r.rots.size() << ' ' << parse_base_conv(r.base_conv).size() << ' ' << r.sud.size() << ' ' << r.pmu.size() << ' '
      << r.rsv.size() << ' ' << r.scalars.size() << ' ' << r.comm_size << ' ' << r.comm_num_limbs << ' ' << r.comm_srcs.size()
      << ' ' << r.comm_dests.size() << ' ' << call_args << ' ' << (r.function_name.empty() ? "-" : r.function_name) << '\n';
  }
  const std::string text = s.str();
  if (buf && buf_bytes > 0) {
    const size_t n = std::min(text.size(), buf_bytes - 1);
    std::memcpy(buf, text.data(), n);
    buf[n] = 0;
  }
  return CERIUM_OK;
}
