// The fiber scheduler behind cuda_emu.h: every CUDA thread of a block is a ucontext fiber on the calling OS thread.
// A fiber runs until it reaches a rendezvous (block barrier, warp barrier, shuffle, vote) or returns; the scheduler
// then resumes the next fiber that is not finished. A rendezvous completes when every live participant has arrived
// (a thread that has returned from the kernel counts as arrived, as exited threads do for `bar.sync` on the device).
#define NC_EMU
#include "cuda_emu.h"

#include <ucontext.h>

#include <cstdio>
#include <cstdlib>
#include <memory>
#include <utility>
#include <vector>

namespace emu {

namespace {

constexpr size_t kStackBytes = 128 * 1024;

struct Fiber {
  ucontext_t ctx;
  std::unique_ptr<char[]> stack;
  ThreadState state;
  bool done = false;
  int linear = 0;       // thread index inside the block
};

struct Warp {
  uint32_t slot[32];
  bool pred[32];
  int arrived = 0;
  unsigned generation = 0;
};

struct Block {
  std::vector<Fiber> fibers;
  std::vector<Warp> warps;
  ucontext_t scheduler;
  int current = -1;
  int live = 0;
  int barrier_arrived = 0;
  unsigned barrier_generation = 0;
  std::vector<char> shared;
  const std::function<void()>* body = nullptr;
};

// Order in which the runnable fibers of a block are resumed in each pass: 0 ascending thread index, 1 descending,
// 2 a fresh pseudo-random permutation per pass. A kernel whose result depends on the order has a race between
// threads that no barrier orders; running it under several schedules and comparing the outputs finds such races.
int g_schedule_mode = 0;
unsigned long long g_schedule_state = 1;

unsigned NextRandom() {
  g_schedule_state = g_schedule_state * 6364136223846793005ull + 1442695040888963407ull;
  return static_cast<unsigned>(g_schedule_state >> 33);
}

thread_local Block* g_block = nullptr;
thread_local ThreadState g_outside;   // coordinates seen by code that is not inside a launch

void yield_to_scheduler() {
  Block* b = g_block;
  Fiber& f = b->fibers[b->current];
  swapcontext(&f.ctx, &b->scheduler);
}

int live_lanes(const Block& b, int warp, unsigned mask) {
  int n = 0;
  for (int l = 0; l < 32; ++l) {
    const size_t t = static_cast<size_t>(warp) * 32 + l;
    if ((mask >> l & 1u) && t < b.fibers.size() && !b.fibers[t].done) ++n;
  }
  return n;
}

void trampoline() {
  Block* b = g_block;
  (*b->body)();
  Fiber& f = b->fibers[b->current];
  f.done = true;
  --b->live;
  swapcontext(&f.ctx, &b->scheduler);
}

}  // namespace

ThreadState& self() { return g_block != nullptr && g_block->current >= 0 ? g_block->fibers[g_block->current].state : g_outside; }

void sync_block() {
  Block* b = g_block;
  const unsigned gen = b->barrier_generation;
  ++b->barrier_arrived;
  while (b->barrier_generation == gen) {
    if (b->barrier_arrived >= b->live) {     // everyone who can still arrive has arrived
      b->barrier_arrived = 0;
      ++b->barrier_generation;
      break;
    }
    yield_to_scheduler();
  }
}

static void warp_rendezvous(unsigned mask) {
  Block* b = g_block;
  const int warp = b->fibers[b->current].linear >> 5;
  Warp& w = b->warps[warp];
  const unsigned gen = w.generation;
  ++w.arrived;
  while (w.generation == gen) {
    if (w.arrived >= live_lanes(*b, warp, mask)) {
      w.arrived = 0;
      ++w.generation;
      break;
    }
    yield_to_scheduler();
  }
}

void sync_warp(unsigned mask) { warp_rendezvous(mask); }

uint32_t exchange(uint32_t mine, int src_lane, unsigned mask) {
  Block* b = g_block;
  const int t = b->fibers[b->current].linear;
  Warp& w = b->warps[t >> 5];
  w.slot[t & 31] = mine;
  warp_rendezvous(mask);                    // every lane has published
  const uint32_t got = w.slot[src_lane & 31];
  warp_rendezvous(mask);                    // every lane has read: the slots may be overwritten
  return got;
}

unsigned vote(bool pred, unsigned mask) {
  Block* b = g_block;
  const int t = b->fibers[b->current].linear;
  Warp& w = b->warps[t >> 5];
  w.pred[t & 31] = pred;
  warp_rendezvous(mask);
  unsigned bits = 0;
  for (int l = 0; l < 32; ++l) {
    const size_t tt = static_cast<size_t>(t >> 5) * 32 + l;
    if ((mask >> l & 1u) && tt < b->fibers.size() && !b->fibers[tt].done && w.pred[l]) bits |= 1u << l;
  }
  warp_rendezvous(mask);
  return bits;
}

void* dynamic_shared() { return g_block->shared.data(); }

void launch(Dim grid, Dim block, size_t dynamic_shared_bytes, const std::function<void()>& body) {
  const int threads = static_cast<int>(block.x * block.y * block.z);
  if (threads <= 0 || threads > 1024) {
    std::fprintf(stderr, "emu::launch: %d threads per block\n", threads);
    std::abort();
  }
  Block b;
  b.body = &body;
  b.fibers.resize(static_cast<size_t>(threads));
  for (auto& f : b.fibers) f.stack.reset(new char[kStackBytes]);
  b.warps.resize(static_cast<size_t>((threads + 31) / 32));
  b.shared.assign(dynamic_shared_bytes + 16, 0);
  Block* outer = g_block;
  g_block = &b;
  std::vector<int> order(static_cast<size_t>(threads));
  for (int t = 0; t < threads; ++t) order[static_cast<size_t>(t)] = g_schedule_mode == 1 ? threads - 1 - t : t;
  for (unsigned bz = 0; bz < grid.z; ++bz)
    for (unsigned by = 0; by < grid.y; ++by)
      for (unsigned bx = 0; bx < grid.x; ++bx) {
        b.live = threads;
        b.barrier_arrived = 0;
        for (auto& w : b.warps) w.arrived = 0;
        for (int t = 0; t < threads; ++t) {
          Fiber& f = b.fibers[static_cast<size_t>(t)];
          f.done = false;
          f.linear = t;
          f.state.grid = grid;
          f.state.block_dim = block;
          f.state.block_idx = Dim{bx, by, bz};
          f.state.thread_idx = Dim{static_cast<unsigned>(t) % block.x, (static_cast<unsigned>(t) / block.x) % block.y,
                                   static_cast<unsigned>(t) / (block.x * block.y)};
          getcontext(&f.ctx);
          f.ctx.uc_stack.ss_sp = f.stack.get();
          f.ctx.uc_stack.ss_size = kStackBytes;
          f.ctx.uc_link = &b.scheduler;
          makecontext(&f.ctx, trampoline, 0);
        }
        // round-robin until every fiber has returned; a full pass in which nothing changes is a deadlock
        while (b.live > 0) {
          if (g_schedule_mode == 2) {
            for (int i = threads - 1; i > 0; --i) std::swap(order[static_cast<size_t>(i)], order[NextRandom() % (i + 1)]);
          }
          for (int k = 0; k < threads && b.live > 0; ++k) {
            const int t = order[static_cast<size_t>(k)];
            if (b.fibers[static_cast<size_t>(t)].done) continue;
            b.current = t;
            swapcontext(&b.scheduler, &b.fibers[static_cast<size_t>(t)].ctx);
          }
        }
        b.current = -1;
      }
  g_block = outer;
}

}  // namespace emu

// mode: 0 ascending, 1 descending, 2 random per pass (seeded). Applies to every later launch of this process.
extern "C" void nc_emu_set_schedule(int mode, unsigned long long seed) {
  emu::g_schedule_mode = mode;
  emu::g_schedule_state = seed * 2 + 1;
}
