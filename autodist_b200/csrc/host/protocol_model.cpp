// Host model of the symmetric-memory synchronisation protocol used by the communication kernels.
//
// The device kernels order their phases with two primitives: a cross-rank barrier in which block b of every rank
// meets block b of every other rank through one flag word per (block, sender) carrying an epoch, and a grid barrier
// among the blocks of one rank (arrival count + generation word). This file runs the same state machines with
// std::atomic release / acquire operations, one host thread per (rank, block), so the protocol - epoch arithmetic
// across wrap-around, replay without resetting flags, phase ordering of a packed two-shot all-reduce, and the bounded
// wait that reports which peer never arrived - can be checked on a machine without a GPU.
//
// Nothing here corresponds to code in petuum/autodist, which has no device-side protocol of its own.
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include <algorithm>
#include <atomic>
#include <chrono>
#include <cmath>
#include <cstdint>
#include <memory>
#include <thread>
#include <vector>

namespace py = pybind11;

namespace {

using Clock = std::chrono::steady_clock;

struct RankState {
  std::unique_ptr<std::atomic<uint32_t>[]> flags;   // [block][sender]
  std::vector<uint32_t> epochs;                     // per block, touched by that block's thread only
  std::atomic<uint32_t> grid_count{0}, grid_gen{0};
  std::atomic<int> error{0};
  std::vector<float> grad, wire, out;
};

struct World {
  int world, blocks;
  long long timeout_ns;
  std::vector<std::unique_ptr<RankState>> ranks;
};

bool expired(Clock::time_point t0, long long timeout_ns) {
  return std::chrono::duration_cast<std::chrono::nanoseconds>(Clock::now() - t0).count() > timeout_ns;
}

// Cross-rank barrier of block `b`: publish the new epoch to every peer, then wait until every peer has published an
// epoch that is not behind it. The comparison is done on the signed difference so that it survives 32-bit wrap-around.
bool sym_barrier(World& w, int rank, int b) {
  RankState& me = *w.ranks[rank];
  const uint32_t e = ++me.epochs[b];
  for (int peer = 0; peer < w.world; ++peer)
    w.ranks[peer]->flags[(size_t)b * w.world + rank].store(e, std::memory_order_release);
  bool ok = true;
  for (int peer = 0; peer < w.world; ++peer) {
    const auto t0 = Clock::now();
    uint32_t it = 0;
    while ((int32_t)(me.flags[(size_t)b * w.world + peer].load(std::memory_order_acquire) - e) < 0) {
      if (((++it) & 63u) == 0) {
        if (expired(t0, w.timeout_ns)) {
          me.error.exchange(100 + peer);
          ok = false;
          break;
        }
        std::this_thread::yield();
      }
    }
  }
  return ok;
}

// Barrier among the blocks of one rank: the last arrival resets the count and bumps the generation.
bool grid_barrier(World& w, int rank) {
  RankState& me = *w.ranks[rank];
  const uint32_t gen = me.grid_gen.load(std::memory_order_acquire);
  if (me.grid_count.fetch_add(1, std::memory_order_acq_rel) == (uint32_t)w.blocks - 1) {
    me.grid_count.store(0, std::memory_order_relaxed);
    me.grid_gen.fetch_add(1, std::memory_order_release);
    return true;
  }
  const auto t0 = Clock::now();
  uint32_t it = 0;
  while (me.grid_gen.load(std::memory_order_acquire) == gen) {
    if (((++it) & 63u) == 0) {
      if (expired(t0, w.timeout_ns)) {
        me.error.exchange(300);
        return false;
      }
      std::this_thread::yield();
    }
  }
  return true;
}

// One packed two-shot mean all-reduce as block `b` of `rank` runs it.
void allreduce_block(World& w, int rank, int b, long long n, bool with_grid_barriers) {
  RankState& me = *w.ranks[rank];
  for (long long i = b; i < n; i += w.blocks) me.wire[i] = me.grad[i];                       // pack (block-strided)
  if (with_grid_barriers && !grid_barrier(w, rank)) return;
  if (!sym_barrier(w, rank, b)) return;
  const long long lo = n * rank / w.world, hi = n * (rank + 1) / w.world;                    // the slice this rank owns
  const long long per = (hi - lo + w.blocks - 1) / w.blocks;
  const long long s0 = lo + per * b, s1 = std::min(hi, s0 + per);
  for (long long i = s0; i < s1; ++i) {
    float s = 0.f;
    for (int p = 0; p < w.world; ++p) s += w.ranks[p]->wire[i];
    s /= (float)w.world;
    for (int p = 0; p < w.world; ++p) w.ranks[p]->wire[i] = s;
  }
  if (!sym_barrier(w, rank, b)) return;
  if (with_grid_barriers && !grid_barrier(w, rank)) return;
  for (long long i = b; i < n; i += w.blocks) me.out[i] = me.wire[i];                        // unpack
}

// Runs `iters` all-reduces of `n` elements among `world` ranks of `blocks` blocks each. Ranks listed in `absent`
// never start (a process that died before the step). Returns (per-rank error codes, max abs error of present ranks).
py::tuple simulate_allreduce(int world, int blocks, long long n, int iters, std::vector<int> absent, double timeout_ms,
                             uint32_t first_epoch, bool with_grid_barriers) {
  if (world < 1 || world > 64 || blocks < 1 || blocks > 64 || n < 0 || iters < 1) throw std::invalid_argument("bad sizes");
  World w;
  w.world = world;
  w.blocks = blocks;
  w.timeout_ns = (long long)(timeout_ms * 1e6);
  for (int r = 0; r < world; ++r) {
    auto st = std::make_unique<RankState>();
    st->flags.reset(new std::atomic<uint32_t>[(size_t)blocks * world]);
    for (size_t i = 0; i < (size_t)blocks * world; ++i) st->flags[i].store(first_epoch, std::memory_order_relaxed);
    st->epochs.assign(blocks, first_epoch);
    st->grad.resize(n);
    st->wire.assign(n, 0.f);
    st->out.assign(n, 0.f);
    w.ranks.push_back(std::move(st));
  }
  std::vector<char> is_absent(world, 0);
  for (int r : absent)
    if (r >= 0 && r < world) is_absent[r] = 1;
  double max_err = 0.0;
  {
    py::gil_scoped_release nogil;
    for (int it = 0; it < iters; ++it) {
      for (int r = 0; r < world; ++r)
        for (long long i = 0; i < n; ++i) w.ranks[r]->grad[i] = (float)((r + 1) * ((i + it) % 17) - 3 * r);
      std::vector<std::thread> threads;
      for (int r = 0; r < world; ++r) {
        if (is_absent[r]) continue;
        for (int b = 0; b < blocks; ++b) threads.emplace_back(allreduce_block, std::ref(w), r, b, n, with_grid_barriers);
      }
      for (auto& t : threads) t.join();
      bool failed = false;
      for (int r = 0; r < world; ++r) failed = failed || w.ranks[r]->error.load() != 0;
      if (failed) break;
      for (long long i = 0; i < n; ++i) {
        float ref = 0.f;
        for (int r = 0; r < world; ++r) ref += w.ranks[r]->grad[i];
        ref /= (float)world;
        for (int r = 0; r < world; ++r) max_err = std::max(max_err, (double)std::fabs(w.ranks[r]->out[i] - ref));
      }
    }
  }
  std::vector<int> errors;
  for (int r = 0; r < world; ++r) errors.push_back(w.ranks[r]->error.load());
  return py::make_tuple(errors, max_err);
}

// Bounded-staleness gate: before step s a rank publishes s to every peer and waits until s - (a peer's published step)
// <= staleness for every peer, or until the time limit. Rank r sleeps delays_us[r] per step (the work of the step), so a
// slow rank can be modelled without asserting on wall-clock time: the function returns, per rank, the largest lead
// over the slowest peer that the gate ever let through, and the error codes (200 + the peer waited for).
py::tuple simulate_staleness(int world, int steps, uint32_t staleness, std::vector<int> delays_us, double timeout_ms,
                             std::vector<int> stop_after) {
  if (world < 1 || world > 64 || steps < 1) throw std::invalid_argument("bad sizes");
  delays_us.resize(world, 0);
  stop_after.resize(world, steps);                               // a rank that stops early never publishes later steps
  std::unique_ptr<std::atomic<uint32_t>[]> clocks(new std::atomic<uint32_t>[(size_t)world * world]);   // [owner][sender]
  for (size_t i = 0; i < (size_t)world * world; ++i) clocks[i].store(0, std::memory_order_relaxed);
  std::vector<int> max_lead(world, 0), errors(world, 0), reached(world, 0);
  const long long timeout_ns = (long long)(timeout_ms * 1e6);
  auto run = [&](int rank) {
    for (int s = 1; s <= std::min(steps, stop_after[rank]); ++s) {
      for (int peer = 0; peer < world; ++peer) clocks[(size_t)peer * world + rank].store((uint32_t)s, std::memory_order_release);
      for (int peer = 0; peer < world; ++peer) {
        const auto t0 = Clock::now();
        uint32_t it = 0;
        while ((int32_t)((uint32_t)s - clocks[(size_t)rank * world + peer].load(std::memory_order_acquire)) > (int32_t)staleness) {
          if (((++it) & 63u) == 0) {
            if (expired(t0, timeout_ns)) {
              errors[rank] = 200 + peer;
              return;
            }
            std::this_thread::yield();
          }
        }
      }
      int slowest = s;
      for (int peer = 0; peer < world; ++peer)
        slowest = std::min(slowest, (int)clocks[(size_t)rank * world + peer].load(std::memory_order_acquire));
      max_lead[rank] = std::max(max_lead[rank], s - slowest);
      reached[rank] = s;
      if (delays_us[rank] > 0) std::this_thread::sleep_for(std::chrono::microseconds(delays_us[rank]));
    }
  };
  {
    py::gil_scoped_release nogil;
    std::vector<std::thread> threads;
    for (int r = 0; r < world; ++r) threads.emplace_back(run, r);
    for (auto& t : threads) t.join();
  }
  return py::make_tuple(max_lead, errors, reached);
}

}  // namespace

void register_batch_feeder(py::module& m);      // batch_feeder.cpp

PYBIND11_MODULE(_adb200_host, m) {
  m.doc() = "host-side native components: model of the symmetric-memory barrier protocol, background batch feeder";
  register_batch_feeder(m);
  m.def("simulate_allreduce", &simulate_allreduce, py::arg("world"), py::arg("blocks"), py::arg("n"), py::arg("iters") = 1,
        py::arg("absent") = std::vector<int>{}, py::arg("timeout_ms") = 200.0, py::arg("first_epoch") = 0u,
        py::arg("with_grid_barriers") = true);
  m.def("simulate_staleness", &simulate_staleness, py::arg("world"), py::arg("steps"), py::arg("staleness"),
        py::arg("delays_us") = std::vector<int>{}, py::arg("timeout_ms") = 500.0, py::arg("stop_after") = std::vector<int>{});
}
