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
struct Fiber {
  ucontext_t ctx;
  bool done = false;
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
  unsigned remaining = nthreads;
  while (remaining) {
    for (unsigned t = 0; t < nthreads; t++) {
      Fiber& f = s.fibers[t];
      if (f.done) continue;
      s.current = (int)t;
      t_threadIdx = f.tid;
      swapcontext(&s.sched, &f.ctx);
      if (f.done) remaining--;
    }
  }
}
}  // namespace

unsigned char* dyn_smem() { return t_state->smem.data(); }

void sync_threads() {
  BlockState* s = t_state;
  Fiber& f = s->fibers[s->current];
  swapcontext(&f.ctx, &s->sched);
  t_threadIdx = f.tid;
}

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
