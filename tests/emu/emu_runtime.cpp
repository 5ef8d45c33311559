// Fiber scheduler behind emu_cuda.h.  TEST INFRASTRUCTURE ONLY (see emu_cuda.h).
#include <ucontext.h>

#include <atomic>
#include <vector>

#include "emu_cuda.h"

namespace cerium_emu {

thread_local uint3 t_threadIdx, t_blockIdx;
thread_local dim3 t_blockDim, t_gridDim;

namespace {
constexpr size_t kStack = 128 * 1024;
enum Wait { kNone = 0, kWarp = 1, kBlock = 2 };
struct Fiber {
  ucontext_t ctx;
  bool done = false;
  int wait = kNone;
  uint3 tid;
};
struct BlockState {
  ucontext_t sched;
  std::vector<Fiber> fibers;
  std::vector<char> stacks;
  int current = -1;
  const std::function<void()>* body = nullptr;
  std::vector<unsigned char> smem;
};
thread_local BlockState* t_state = nullptr;
std::atomic<long> g_launches{0};

void fiber_entry() {
  BlockState* s = t_state;
  Fiber& f = s->fibers[s->current];
  (*s->body)();
  f.done = true;
  swapcontext(&f.ctx, &s->sched);
}

void run_block(BlockState& s, dim3 block, const std::function<void()>& body) {
  const unsigned nthreads = block.x * block.y * block.z;
  s.fibers.assign(nthreads, Fiber());
  if (s.stacks.size() < (size_t)nthreads * kStack) s.stacks.resize((size_t)nthreads * kStack);
  s.body = &body;
  t_state = &s;
  for (unsigned t = 0; t < nthreads; t++) {
    Fiber& f = s.fibers[t];
    f.tid = uint3{t % block.x, (t / block.x) % block.y, t / (block.x * block.y)};
    getcontext(&f.ctx);
    f.ctx.uc_stack.ss_sp = s.stacks.data() + (size_t)t * kStack;
    f.ctx.uc_stack.ss_size = kStack;
    f.ctx.uc_link = &s.sched;
    makecontext(&f.ctx, fiber_entry, 0);
  }
  // Scheduling: repeatedly pick a warp at (seeded) random and advance its 32 fibers by one phase,
  // i.e. to their next barrier or their end.  __syncwarp() holds only the fibers of one warp
  // together, __syncthreads() parks the warp until every warp has arrived.  Random interleaving of
  // warp phases is a legal GPU schedule, and it makes code that needs a block barrier where it only
  // has a warp barrier compute wrong results here as well.
  unsigned remaining = nthreads;
  const unsigned nwarps = (nthreads + 31) / 32;
  std::vector<int> state(nwarps, kNone);  // kNone = runnable, kBlock = parked, -1 = finished
  uint64_t rng = 0x9E3779B97F4A7C15ull ^ ((uint64_t)t_blockIdx.x << 32) ^ t_blockIdx.y;
  while (remaining) {
    std::vector<unsigned> runnable;
    for (unsigned w = 0; w < nwarps; w++)
      if (state[w] == kNone) runnable.push_back(w);
    if (runnable.empty()) {
      for (unsigned w = 0; w < nwarps; w++)
        if (state[w] == kBlock) state[w] = kNone;
      for (unsigned t = 0; t < nthreads; t++)
        if (s.fibers[t].wait == kBlock) s.fibers[t].wait = kNone;
      continue;
    }
    rng = rng * 6364136223846793005ull + 1442695040888963407ull;
    const unsigned w = runnable[(rng >> 33) % runnable.size()];
    const unsigned lo = w * 32, hi = lo + 32 < nthreads ? lo + 32 : nthreads;
    bool all_done = true, parked = false;
    for (unsigned t = lo; t < hi; t++) {
      Fiber& f = s.fibers[t];
      if (f.done) continue;
      f.wait = kNone;
      s.current = (int)t;
      t_threadIdx = f.tid;
      swapcontext(&s.sched, &f.ctx);
      if (f.done) remaining--;
      else {
        all_done = false;
        if (f.wait == kBlock) parked = true;
      }
    }
    state[w] = all_done ? -1 : (parked ? kBlock : kNone);
  }
}
}  // namespace

unsigned char* dyn_smem() { return t_state->smem.data(); }

static void yield_with(int kind) {
  BlockState* s = t_state;
  Fiber& f = s->fibers[s->current];
  f.wait = kind;
  swapcontext(&f.ctx, &s->sched);
  t_threadIdx = f.tid;
}
void sync_threads() { yield_with(kBlock); }
void sync_warp() { yield_with(kWarp); }

long launches() { return g_launches.load(); }

void launch(dim3 grid, dim3 block, size_t smem_bytes, const std::function<void()>& body) {
  g_launches++;
  const long nblocks = (long)grid.x * grid.y * grid.z;
#pragma omp parallel
  {
    BlockState state;
    state.smem.resize(smem_bytes + 16);
    t_blockDim = block;
    t_gridDim = grid;
#pragma omp for schedule(dynamic, 1)
    for (long b = 0; b < nblocks; b++) {
      t_blockIdx = uint3{(unsigned)(b % grid.x), (unsigned)((b / grid.x) % grid.y), (unsigned)(b / ((long)grid.x * grid.y))};
      run_block(state, block, body);
    }
    t_state = nullptr;
  }
}

}  // namespace cerium_emu
