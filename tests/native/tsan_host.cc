// Race-detection driver for the host runtime: built with -fsanitize=thread (no OpenMP) and run by the test suite.
// Exercises every place where host threads share state: mailbox and TCP transports with the ring all-reduce,
// the mesh runtime's replica threads, and the data loader's prefetch thread.
#include <cmath>
#include <cstdio>
#include <thread>
#include <vector>

#include "collective.h"
#include "core.h"
#include "mesh.h"

using namespace ncb;

static int Check(bool ok, const char* what) {
  if (!ok) std::fprintf(stderr, "FAILED: %s\n", what);
  return ok ? 0 : 1;
}

int main() {
  int bad = 0;
  {  // ring over mailboxes
    const int world = 4, count = 1001;
    MemoryHub hub(world);
    std::vector<std::vector<float>> data(world, std::vector<float>(count));
    for (int r = 0; r < world; ++r)
      for (int i = 0; i < count; ++i) data[r][i] = static_cast<float>(r + 1) * 0.5f + static_cast<float>(i % 7);
    std::vector<std::thread> th;
    std::vector<char> ok(world, 0);
    for (int r = 0; r < world; ++r)
      th.emplace_back([&, r] {
        auto link = hub.Endpoint(r);
        ok[r] = RingAllReduceSum(link.get(), data[r].data(), count, 10000);
      });
    for (auto& t : th) t.join();
    for (int r = 0; r < world; ++r) bad += Check(ok[r] && data[r] == data[0], "memory ring");
    bad += Check(std::fabs(data[0][3] - (5.0f + 4 * 3.0f)) < 1e-5f, "memory ring value");
  }
  {  // ring over TCP, three ranks as threads
    const int world = 3, count = 70000;  // larger than a socket buffer: the sender thread must keep draining
    std::vector<std::unique_ptr<TcpTransport>> links;
    std::vector<int> ports;
    for (int r = 0; r < world; ++r) {
      links.push_back(std::make_unique<TcpTransport>(r, world));
      ports.push_back(links.back()->port());
    }
    std::vector<std::vector<float>> data(world, std::vector<float>(count, 1.0f));
    std::vector<char> ok(world, 0);
    std::vector<std::thread> th;
    for (int r = 0; r < world; ++r)
      th.emplace_back([&, r] {
        ok[r] = links[r]->Connect(ports, 10000) && RingAllReduceSum(links[r].get(), data[r].data(), count, 10000);
      });
    for (auto& t : th) t.join();
    for (int r = 0; r < world; ++r) bad += Check(ok[r] && data[r][0] == 3.0f && data[r][count - 1] == 3.0f, "tcp ring");
  }
  {  // mesh runtime: two replica threads, two steps
    EngineConfig cfg;
    cfg.num_layers = 2, cfg.num_heads = 2, cfg.num_kv_heads = 2, cfg.hidden_dim = 32, cfg.seq_len = 16;
    cfg.vocab_size = 64, cfg.padded_vocab_size = 64, cfg.window_pattern = "SL";
    MeshSpec mesh;
    mesh.devices = {0, 1};
    std::string err;
    MeshRuntime rt(mesh, cfg, OptimConfig(), 4, 1, 0, 7, &err);
    bad += Check(rt.ok(), "mesh create");
    std::vector<int> tok(4 * 16), tgt(4 * 16);
    for (std::size_t i = 0; i < tok.size(); ++i) tok[i] = static_cast<int>((i * 7 + 3) % 64), tgt[i] = static_cast<int>((i * 5 + 1) % 64);
    for (int s = 0; s < 2; ++s) {
      const float loss = rt.TrainStep(tok.data(), tgt.data(), &err);
      bad += Check(rt.ok() && loss > 0.0f, "mesh step");
    }
    bad += Check(rt.ParamDigest(0) == rt.ParamDigest(1), "replica digests");
  }
  {  // loader prefetch thread
    auto loader = std::make_unique<DataLoader>(ZipfSource(64, 40, 1.1, 5), 2, 16, 32, 2, 1);
    std::vector<int> a(32), b(32);
    for (int i = 0; i < 20; ++i) loader->Next(a.data(), b.data());
    const LoaderState st = loader->State();
    (void)st;
  }
  std::printf(bad ? "tsan driver: %d checks failed\n" : "tsan driver: ok\n", bad);
  return bad ? 1 : 0;
}
