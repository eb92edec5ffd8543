// Launches one generated kernel on host threads (see shim.h).
#include <algorithm>
#include <condition_variable>
#include <mutex>
#include <thread>
#include <vector>

#include "shim.h"

namespace emu {
namespace {
struct Barrier {
  std::mutex m;
  std::condition_variable cv;
  int expected = 0, waiting = 0;
  unsigned gen = 0;
  void reset(int n) { expected = n; waiting = 0; }
  void wait() {
    std::unique_lock<std::mutex> l(m);
    const unsigned g = gen;
    if (++waiting >= expected) { waiting = 0; gen++; cv.notify_all(); }
    else cv.wait(l, [&] { return gen != g; });
  }
  void drop() {                       // a thread that has returned no longer takes part
    std::unique_lock<std::mutex> l(m);
    expected--;
    if (expected > 0 && waiting >= expected) { waiting = 0; gen++; cv.notify_all(); }
  }
};
struct Warp {
  Barrier bar;
  unsigned long long buf[32];
  int lanes = 32;
};
thread_local Warp* t_warp = nullptr;
Barrier g_block_bar;
}  // namespace
thread_local Dim t_thread, t_block;
thread_local int t_lane = 0;
Dim g_block_dim, g_grid_dim;

void block_barrier() { g_block_bar.wait(); }
void warp_barrier() { t_warp->bar.wait(); }
int warp_lanes() { return t_warp->lanes; }
unsigned long long warp_exchange(unsigned long long value, int src) {
  Warp& w = *t_warp;
  w.buf[t_lane] = value;
  w.bar.wait();
  const unsigned long long got = w.buf[(src >= 0 && src < w.lanes) ? src : t_lane];
  w.bar.wait();
  return got;
}
unsigned warp_ballot(int pred) {
  Warp& w = *t_warp;
  w.buf[t_lane] = pred ? 1ull : 0ull;
  w.bar.wait();
  unsigned r = 0;
  for (int l = 0; l < w.lanes; l++) r |= (unsigned)(w.buf[l] & 1ull) << l;
  w.bar.wait();
  return r;
}
}  // namespace emu

namespace {
typedef void* P;
// Every kernel parameter is a pointer. With the C calling convention of x86-64 and AArch64 a callee ignores arguments
// it does not declare, so one call shape with 64 pointers serves every kernel (the rest are null).
void call(void* fn, int n, void** a) {
  if (n > 64) std::terminate();
  P p[64] = {};
  for (int k = 0; k < n; k++) p[k] = a[k];
  ((void (*)(P, P, P, P, P, P, P, P, P, P, P, P, P, P, P, P, P, P, P, P, P, P, P, P, P, P, P, P, P, P, P, P, P, P, P, P, P, P, P, P, P, P, P, P, P, P, P, P, P, P, P, P, P, P, P, P, P, P, P, P, P, P, P, P))fn)(p[0], p[1], p[2], p[3], p[4], p[5], p[6], p[7], p[8], p[9], p[10], p[11], p[12], p[13], p[14], p[15], p[16], p[17], p[18], p[19], p[20], p[21], p[22], p[23], p[24], p[25], p[26], p[27], p[28], p[29], p[30], p[31], p[32], p[33], p[34], p[35], p[36], p[37], p[38], p[39], p[40], p[41], p[42], p[43], p[44], p[45], p[46], p[47], p[48], p[49], p[50], p[51], p[52], p[53], p[54], p[55], p[56], p[57], p[58], p[59], p[60], p[61], p[62], p[63]);
}
}  // namespace

extern "C" void emu_launch(void* fn, int nargs, void** args, int gx, int gy, int gz, int bx, int by, int bz) {
  using namespace emu;
  const int nthreads = bx * by * bz, nwarps = (nthreads + 31) / 32;
  g_block_dim = {(unsigned)bx, (unsigned)by, (unsigned)bz};
  g_grid_dim = {(unsigned)gx, (unsigned)gy, (unsigned)gz};
  std::vector<Warp> warps(nwarps);
  Barrier rendezvous;
  rendezvous.reset(nthreads);
  const long long blocks = (long long)gx * gy * gz;
  auto arm = [&]() {
    g_block_bar.reset(nthreads);
    for (int w = 0; w < nwarps; w++) {
      warps[w].lanes = std::min(32, nthreads - 32 * w);
      warps[w].bar.reset(warps[w].lanes);
    }
  };
  arm();
  std::vector<std::thread> team;
  for (int t = 0; t < nthreads; t++) {
    team.emplace_back([&, t]() {
      t_thread = {(unsigned)(t % bx), (unsigned)((t / bx) % by), (unsigned)(t / (bx * by))};
      t_warp = &warps[t / 32];
      t_lane = t % 32;
      for (long long b = 0; b < blocks; b++) {
        t_block = {(unsigned)(b % gx), (unsigned)((b / gx) % gy), (unsigned)(b / ((long long)gx * gy))};
        call(fn, nargs, args);
        g_block_bar.drop();           // an exited thread no longer takes part in the block's barriers
        t_warp->bar.drop();
        rendezvous.wait();            // the block is over for everyone
        if (t == 0) arm();
        rendezvous.wait();
      }
    });
  }
  for (auto& th : team) th.join();
}
