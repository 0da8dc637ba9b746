// Threaded host twin of the expert-parallel MoE step: the synchronisation structure of
// splits_scan / dispatch_push / gated grouped GEMMs / peer_signal / combine_pull and of the backward
// pass (fast_b200/parallel/ep.py, csrc/kernels/moe_route.cu, moe_comm.cu), with std::atomic for
// every flag and counter and plain memory for every payload buffer that peers read or write.
// One thread per rank plays the stream (kernels in order, each kernel = a few worker threads that
// are joined at its end); ranks are never synchronised with each other except through the
// protocol's own flags. Consecutive steps reuse every buffer, which is the point: built with
// -fsanitize=thread (build/fastb-moe-twin-tsan) any reuse that the count exchange, the arrival
// counters and the ready flags do not order is reported as a data race. Results are also checked
// against values computed directly from the routing. Forward-only runs are repeated with the fp8
// receive path (quantised buffer written by peers, converted locally after all experts arrived)
// and with the dispatch overlapped with the gated GEMMs on a side stream, and once more with arrivals
// counted and gated per tile of the receive buffer (the forward-only layer's scheme), including the
// direct read of the quantised rows by the GEMM.
#include <atomic>
#include <cstdint>
#include <cstdio>
#include <cstdlib>
#include <functional>
#include <memory>
#include <thread>
#include <vector>

namespace {

constexpr int H = 4;        // words per row
constexpr int RA = 4;       // group rows are padded to a multiple of this
constexpr int kWorkers = 3;

struct Cfg { int W, El, K, T, steps; bool training; bool bwd_entry_handshake; bool fp8 = false; bool overlap = false; bool tiles = false; };

uint64_t mix(uint64_t x) { x += 0x9e3779b97f4a7c15ull; x = (x ^ (x >> 30)) * 0xbf58476d1ce4e5b9ull; x = (x ^ (x >> 27)) * 0x94d049bb133111ebull; return x ^ (x >> 31); }

struct Rank {
  // symmetric (peers touch these)
  std::vector<int> counts;                                // [W][E] plain: written by peers' split scans
  std::unique_ptr<std::atomic<uint64_t>[]> flags;         // [4][W]: 0 counts, 1 y ready, 2 bwd entry, 3 dx ready
  std::unique_ptr<std::atomic<uint64_t>[]> arrive;        // [2][El] monotone row counters
  std::unique_ptr<std::atomic<uint64_t>[]> tile_arrive;   // [cap / RA] monotone row counters per tile of RA rows (forward-only layer)
  std::vector<uint64_t> tile_target;                      // [cap / RA] local
  std::vector<uint32_t> x_recv, y, dy_recv, dx_recv;      // [cap][H] plain
  std::vector<uint32_t> xq_recv;                          // [cap][H] plain: quantised rows (fp8 dispatch); x_recv is then local
  // local
  std::vector<uint64_t> target;                           // [2][El]
  std::vector<int> send_base, group_off, group_rows;      // [E], [El + 1], [El]
  std::vector<uint32_t> gu;                               // [cap][H] saved activation (local only)
};

struct World {
  Cfg c; int E, cap;
  std::vector<std::unique_ptr<Rank>> r;
  std::atomic<int> failures{0};
  std::atomic<int> abort{0};
};

bool wait_ge(World& w, const std::atomic<uint64_t>& f, uint64_t want) {
  unsigned spins = 0;
  while (f.load(std::memory_order_acquire) < want) {
    if ((++spins & 1023u) == 0u) {
      if (w.abort.load(std::memory_order_acquire)) return false;
      std::this_thread::yield();
    }
    if (spins > (1u << 30)) { w.abort.store(1); w.failures.fetch_add(1); std::printf("FAIL: wait ran out\n"); return false; }
  }
  return true;
}

void parallel(int n, const std::function<void(int, int)>& body) {  // one "kernel": workers joined at its end
  std::vector<std::thread> ts;
  for (int k = 0; k < n; ++k) ts.emplace_back(body, k, n);
  for (auto& t : ts) t.join();
}

uint32_t x_word(int rank, int step, int t, int i) { return static_cast<uint32_t>(mix((static_cast<uint64_t>(rank) << 40) ^ (static_cast<uint64_t>(step) << 24) ^ (t << 4) ^ i) & 0xffff); }
uint32_t g_word(int rank, int step, int t, int i) { return static_cast<uint32_t>(mix(0x5555ull ^ (static_cast<uint64_t>(rank) << 40) ^ (static_cast<uint64_t>(step) << 24) ^ (t << 4) ^ i) & 0xffff); }

void run_rank(World& w, int me) {
  const Cfg& c = w.c;
  const int W = c.W, El = c.El, E = w.E, K = c.K, T = c.T;
  Rank& my = *w.r[me];
  std::vector<int> topk(static_cast<size_t>(T) * K), dest_row(static_cast<size_t>(T) * K);
  for (int step = 1; step <= c.steps && !w.abort.load(); ++step) {
    const uint64_t epoch = static_cast<uint64_t>(step);
    // ---- routing (local): K distinct experts per token -------------------------------------------
    std::vector<int> mine(E, 0);
    for (int t = 0; t < T; ++t) {
      const int first = static_cast<int>(mix((static_cast<uint64_t>(me) << 32) ^ (static_cast<uint64_t>(step) << 16) ^ t) % E);
      int hop = 1 + static_cast<int>(mix(first + 77ull * t + step) % E);  // coprime with E => K distinct experts
      auto gcd = [](int a, int b) { while (b) { const int r = a % b; a = b; b = r; } return a; };
      while (gcd(hop, E) != 1) hop = hop % E + 1;
      for (int j = 0; j < K; ++j) topk[t * K + j] = (first + j * hop) % E;
      for (int j = 0; j < K; ++j) ++mine[topk[t * K + j]];
    }
    // ---- splits_scan: count all-gather by stores, flag, wait, derive offsets ---------------------
    for (int p = 0; p < W; ++p)
      for (int e = 0; e < E; ++e) w.r[p]->counts[static_cast<size_t>(me) * E + e] = mine[e];
    for (int p = 0; p < W; ++p) w.r[p]->flags[0 * W + me].store(epoch, std::memory_order_release);
    for (int p = 0; p < W; ++p) if (!wait_ge(w, my.flags[0 * W + p], epoch)) return;
    std::vector<int> tot(E, 0), padded(E, 0), before(E, 0);
    for (int e = 0; e < E; ++e) {
      for (int s = 0; s < W; ++s) { const int cnt = my.counts[static_cast<size_t>(s) * E + e]; tot[e] += cnt; if (s < me) before[e] += cnt; }
      padded[e] = (tot[e] + RA - 1) / RA * RA;
    }
    for (int e = 0; e < E; ++e) {
      const int d = e / El, le = e % El;
      int base = 0;
      for (int q = 0; q < le; ++q) base += padded[d * El + q];
      my.send_base[e] = base + before[e];
      if (d == me) {
        my.group_off[le] = base; my.group_rows[le] = tot[e];
        if (le == El - 1) my.group_off[El] = base + padded[e];
        for (int ch = 0; ch < (c.training ? 2 : 1); ++ch) my.target[ch * El + le] += static_cast<uint64_t>(tot[e]);
        if (c.tiles)  // the same per tile: this expert's rows fill its tiles from `base` on
          for (int r0 = 0; r0 < tot[e]; r0 += RA) my.tile_target[(base + r0) / RA] += static_cast<uint64_t>(tot[e] - r0 < RA ? tot[e] - r0 : RA);
      }
    }
    if (my.group_off[El] > w.cap) { w.failures.fetch_add(1); w.abort.store(1); std::printf("FAIL: capacity\n"); return; }
    {  // destination rows: my tokens for expert e are consecutive from send_base[e], in token order
      std::vector<int> next(E, 0);
      for (int t = 0; t < T; ++t)
        for (int j = 0; j < K; ++j) { const int e = topk[t * K + j]; dest_row[t * K + j] = my.send_base[e] + next[e]++; }
    }
    auto zero_pad = [&](std::vector<uint32_t>& buf) {
      for (int le = 0; le < El; ++le)
        for (int row = my.group_off[le] + my.group_rows[le]; row < my.group_off[le + 1]; ++row)
          for (int i = 0; i < H; ++i) buf[static_cast<size_t>(row) * H + i] = 0;
    };
    // ---- dispatch_push (forward): rows straight into the owners' receive buffer, then arrival counts --
    // fp8 mode: peers write the quantised buffer; the owner waits for all its experts, converts into
    // its (then purely local) x_recv and runs the GEMMs ungated. overlap mode: the dispatch runs on a
    // side stream at the same time as the gated GEMMs of the main stream.
    if (!c.fp8) zero_pad(my.x_recv);
    const int ntiles = w.cap / RA;
    auto dispatch = [&](int k, int n) {
      std::vector<int> sent(E, 0);
      std::vector<int> sent_tile(c.tiles ? static_cast<size_t>(W) * ntiles : 0, 0);  // the kernel's per-CTA histogram of destination tiles
      // Tile counts are published (release) and cleared every few tokens, as the sorted dispatch does every few
      // rounds, and once more at the end.
      auto publish_tiles = [&]() {
        for (int p = 0; p < W; ++p)
          for (int tl = 0; tl < ntiles; ++tl) {
            int& cnt = sent_tile[static_cast<size_t>(p) * ntiles + tl];
            if (cnt) { w.r[p]->tile_arrive[tl].fetch_add(static_cast<uint64_t>(cnt), std::memory_order_release); cnt = 0; }
          }
      };
      int rounds = 0;
      for (int t = k; t < T; t += n) {
        for (int j = 0; j < K; ++j) {
          const int e = topk[t * K + j];
          Rank& owner = *w.r[e / El];
          uint32_t* dst = (c.fp8 ? owner.xq_recv : owner.x_recv).data() + static_cast<size_t>(dest_row[t * K + j]) * H;
          for (int i = 0; i < H; ++i) dst[i] = x_word(me, step, t, i) ^ (c.fp8 ? 0x5a5a0000u : 0u);
          ++sent[e];
          if (c.tiles) ++sent_tile[static_cast<size_t>(e / El) * ntiles + dest_row[t * K + j] / RA];
        }
        if (c.tiles && ++rounds % 3 == 0) publish_tiles();
      }
      if (c.tiles) {
        publish_tiles();
        return;
      }
      for (int e = 0; e < E; ++e)
        if (sent[e]) w.r[e / El]->arrive[0 * El + e % El].fetch_add(static_cast<uint64_t>(sent[e]), std::memory_order_release);
    };
    auto gemms = [&](int k, int n) {
      if (c.tiles) {
        // Tile-gated first GEMM of the forward-only layer: a worker takes tiles of RA rows round robin and waits only
        // for the tile it is about to read. With fp8 it reads the quantised rows directly (the converter warps'
        // role) and counts rows past the group's real end as zeros.
        int tile_no = 0;
        for (int le = 0; le < El; ++le)
          for (int row0 = my.group_off[le]; row0 < my.group_off[le + 1]; row0 += RA, ++tile_no) {
            if (tile_no % n != k) continue;
            if (!wait_ge(w, my.tile_arrive[row0 / RA], my.tile_target[row0 / RA])) return;
            for (int row = row0; row < row0 + RA; ++row)
              for (int i = 0; i < H; ++i) {
                const bool live = row < my.group_off[le] + my.group_rows[le];
                const uint32_t v = !live ? 0u : c.fp8 ? my.xq_recv[static_cast<size_t>(row) * H + i] ^ 0x5a5a0000u : my.x_recv[static_cast<size_t>(row) * H + i];
                my.y[static_cast<size_t>(row) * H + i] = v * 3 + static_cast<uint32_t>(me * El + le + 1);
              }
          }
        return;
      }
      for (int le = k; le < El; le += n) {
        if (!c.fp8 && !wait_ge(w, my.arrive[0 * El + le], my.target[0 * El + le])) return;
        for (int row = my.group_off[le]; row < my.group_off[le + 1]; ++row)
          for (int i = 0; i < H; ++i) {
            const uint32_t v = my.x_recv[static_cast<size_t>(row) * H + i];
            my.gu[static_cast<size_t>(row) * H + i] = v + 7;
            my.y[static_cast<size_t>(row) * H + i] = v * 3 + static_cast<uint32_t>(me * El + le + 1);
          }
      }
    };
    std::thread side;
    if (c.overlap) side = std::thread([&] { parallel(kWorkers, dispatch); });
    else parallel(kWorkers, dispatch);
    if (c.fp8 && !c.tiles) {
      // wait_counters + dequant: all local experts complete, then quantised rows -> x_recv (real rows only), pad rows zeroed
      bool ok = true;
      for (int le = 0; le < El && ok; ++le) ok = wait_ge(w, my.arrive[0 * El + le], my.target[0 * El + le]);
      if (ok)
        for (int le = 0; le < El; ++le)
          for (int row = my.group_off[le]; row < my.group_off[le] + my.group_rows[le]; ++row)
            for (int i = 0; i < H; ++i) my.x_recv[static_cast<size_t>(row) * H + i] = my.xq_recv[static_cast<size_t>(row) * H + i] ^ 0x5a5a0000u;
      zero_pad(my.x_recv);
    }
    parallel(kWorkers, gemms);
    if (side.joinable()) side.join();  // the main stream re-joins the side stream before it signals
    if (w.abort.load()) return;
    for (int p = 0; p < W; ++p) w.r[p]->flags[1 * W + me].store(epoch, std::memory_order_release);  // peer_signal: my y is complete
    // ---- combine_pull: every token pulls its K rows from the owners and sums them ------------------
    auto pull = [&](int flag_row, bool from_dx, const std::function<uint32_t(int, int, int)>& expect) {
#ifndef FASTB_MOE_TWIN_NO_READY_WAIT  // defining it drops the wait for the owners' ready flags: the race detector must object
      for (int p = 0; p < W; ++p) if (!wait_ge(w, my.flags[flag_row * W + p], epoch)) return;
#endif
      parallel(kWorkers, [&](int k, int n) {
        for (int t = k; t < T; t += n)
          for (int i = 0; i < H; ++i) {
            uint32_t acc = 0, want = 0;
            for (int j = 0; j < K; ++j) {
              const int e = topk[t * K + j];
              const Rank& owner = *w.r[e / El];
              const std::vector<uint32_t>& src = from_dx ? owner.dx_recv : owner.y;
              acc += src[static_cast<size_t>(dest_row[t * K + j]) * H + i];
              want += expect(t, j, i);
            }
            if (acc != want) { w.failures.fetch_add(1); if (!w.abort.exchange(1)) std::printf("FAIL: rank %d step %d token %d: got %u want %u\n", me, step, t, acc, want); }
          }
      });
    };
    auto y_expect = [&](int t, int j, int i) { return x_word(me, step, t, i) * 3 + static_cast<uint32_t>(topk[t * K + j] + 1); };
    pull(1, false, y_expect);
    if (!c.training || w.abort.load()) continue;
    // ---- backward: router-weight gradients read y again (still in place on the owners) --------------
    pull(1, false, y_expect);
    // ---- transposed combine: push grad rows to the owners (second arrival channel) ------------------
    zero_pad(my.dy_recv);
    if (c.bwd_entry_handshake) {
      for (int p = 0; p < W; ++p) w.r[p]->flags[2 * W + me].store(epoch, std::memory_order_release);
      for (int p = 0; p < W; ++p) if (!wait_ge(w, my.flags[2 * W + p], epoch)) return;
    }
    parallel(kWorkers, [&](int k, int n) {
      std::vector<int> sent(E, 0);
      for (int t = k; t < T; t += n)
        for (int j = 0; j < K; ++j) {
          const int e = topk[t * K + j];
          uint32_t* dst = w.r[e / El]->dy_recv.data() + static_cast<size_t>(dest_row[t * K + j]) * H;
          for (int i = 0; i < H; ++i) dst[i] = g_word(me, step, t, i) + static_cast<uint32_t>(j);
          ++sent[e];
        }
      for (int e = 0; e < E; ++e)
        if (sent[e]) w.r[e / El]->arrive[1 * El + e % El].fetch_add(static_cast<uint64_t>(sent[e]), std::memory_order_release);
    });
    // ---- dgrad / wgrad: read dy_recv, the saved activations and x_recv; write dx_recv ---------------
    parallel(kWorkers, [&](int k, int n) {
      for (int le = k; le < El; le += n) {
        if (!wait_ge(w, my.arrive[1 * El + le], my.target[1 * El + le])) return;
        for (int row = my.group_off[le]; row < my.group_off[le + 1]; ++row)
          for (int i = 0; i < H; ++i) {
            const size_t at = static_cast<size_t>(row) * H + i;
            my.dx_recv[at] = my.dy_recv[at] * 2 + my.gu[at] + my.x_recv[at];
          }
      }
    });
    if (w.abort.load()) return;
    for (int p = 0; p < W; ++p) w.r[p]->flags[3 * W + me].store(epoch, std::memory_order_release);  // my dx is complete
    // ---- transposed dispatch: every token pulls and sums the gradients of its K rows -----------------
    pull(3, true, [&](int t, int j, int i) { const uint32_t x = x_word(me, step, t, i); return (g_word(me, step, t, i) + static_cast<uint32_t>(j)) * 2 + (x + 7) + x; });
  }
}

int run(const Cfg& c) {
  World w;
  w.c = c; w.E = c.W * c.El;
  w.cap = ((c.W * c.T * (c.K < c.El ? c.K : c.El) + RA * c.El) + RA - 1) / RA * RA;
  for (int r = 0; r < c.W; ++r) {
    auto k = std::make_unique<Rank>();
    k->counts.assign(static_cast<size_t>(c.W) * w.E, 0);
    k->flags.reset(new std::atomic<uint64_t>[4 * c.W]);
    k->arrive.reset(new std::atomic<uint64_t>[2 * c.El]);
    k->tile_arrive.reset(new std::atomic<uint64_t>[w.cap / RA]);
    for (int i = 0; i < w.cap / RA; ++i) k->tile_arrive[i].store(0);
    k->tile_target.assign(w.cap / RA, 0);
    for (int i = 0; i < 4 * c.W; ++i) k->flags[i].store(0);
    for (int i = 0; i < 2 * c.El; ++i) k->arrive[i].store(0);
    for (auto* b : {&k->x_recv, &k->xq_recv, &k->y, &k->dy_recv, &k->dx_recv, &k->gu}) b->assign(static_cast<size_t>(w.cap) * H, 0);
    k->target.assign(2 * c.El, 0);
    k->send_base.assign(w.E, 0); k->group_off.assign(c.El + 1, 0); k->group_rows.assign(c.El, 0);
    w.r.push_back(std::move(k));
  }
  std::vector<std::thread> streams;
  for (int r = 0; r < c.W; ++r) streams.emplace_back(run_rank, std::ref(w), r);
  for (auto& t : streams) t.join();
  return w.failures.load();
}

}  // namespace

int main(int argc, char** argv) {
  const int steps = argc > 1 ? std::atoi(argv[1]) : 4;
  const bool no_handshake = argc > 2 && std::atoi(argv[2]) == 0;
  int runs = 0, failures = 0;
  for (int W : {1, 2, 4})
    for (int El : {1, 2, 3})
      for (int K : {1, 2})
        for (bool training : {false, true}) {
          if (K > W * El) continue;
          Cfg c{W, El, K, 10 + 3 * W, steps, training, !no_handshake};
          failures += run(c);
          ++runs;
          if (!training) {  // the forward-only variants: fp8 receive path, dispatch overlapped with the gated GEMMs
            Cfg f = c; f.fp8 = true;
            failures += run(f);
            Cfg o = c; o.overlap = true;
            failures += run(o);
            Cfg t1 = c; t1.tiles = true;                     // arrivals counted and gated per tile
            failures += run(t1);
            Cfg t2 = c; t2.tiles = true; t2.fp8 = true;      // ... with the quantised rows read by the GEMM itself
            failures += run(t2);
            Cfg t3 = c; t3.tiles = true; t3.overlap = true;  // ... with the dispatch on a side stream
            failures += run(t3);
            runs += 5;
          }
        }
  std::printf("{\"twin_check\":\"moe step protocol\",\"runs\":%d,\"steps\":%d,\"failures\":%d}\n", runs, steps, failures);
  return failures ? 1 : 0;
}
