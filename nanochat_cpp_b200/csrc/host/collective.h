// Host-side collectives for the CPU engine and the control plane: point-to-point transports between the ranks of
// one job on one host, and the ring all-reduce / all-gather built on them.
//
// The reference reduces gradients with a ring over a `Transport` seam (backends/cuda/collective/transport.h:1-132,
// ring_schedule.cc:71-160) whose implementations are an in-process mailbox for tests (memory_transport.*) and TCP
// over 127.0.0.1 with a 16-byte frame header and a sender thread (host_transport.cc:26-201). The GPU path of this
// framework does not use any of this (it reduces through NVLink peer memory, or NCCL); these classes serve the
// native CPU engine's in-process mesh, multi-process CPU jobs, and the rendezvous byte exchange.
#pragma once
#include <atomic>
#include <condition_variable>
#include <cstddef>
#include <cstdint>
#include <deque>
#include <memory>
#include <mutex>
#include <string>
#include <thread>
#include <vector>

namespace ncb {

// Ordered, reliable byte messages between ranks. `Send` never blocks on the receiver (it queues); `Recv` blocks
// until a message of exactly `bytes` from `from` arrives or `timeout_ms` passes (false: peer lost or size mismatch).
class Transport {
 public:
  virtual ~Transport() = default;
  virtual int rank() const = 0;
  virtual int world() const = 0;
  virtual bool Send(int to, const void* data, std::size_t bytes) = 0;
  virtual bool Recv(int from, void* data, std::size_t bytes, int timeout_ms) = 0;
  const std::string& error() const { return error_; }

 protected:
  std::string error_;
};

// In-process mailboxes shared by the endpoints of one job (one endpoint per thread-rank).
class MemoryHub {
 public:
  explicit MemoryHub(int world);
  int world() const { return world_; }
  std::unique_ptr<Transport> Endpoint(int rank);
  // Test hook: the next `count` messages from `from` to `to` are dropped (a lost peer as the receiver sees it).
  void DropNext(int from, int to, int count);

 private:
  friend class MemoryTransport;
  struct Box {
    std::mutex mu;
    std::condition_variable cv;
    std::deque<std::vector<std::uint8_t>> q;
    int drop = 0;
  };
  Box& box(int from, int to) { return *boxes_[static_cast<std::size_t>(from) * world_ + to]; }
  int world_;
  std::vector<std::unique_ptr<Box>> boxes_;
};

// TCP over 127.0.0.1. Every rank listens on an ephemeral port; after the ports have been exchanged (by any
// side channel: a file, a store, the parent process) `Connect` opens one socket per peer pair (the lower rank
// accepts). Frames carry a 16-byte header {magic, sender, byte count}; a sender thread drains the send queue so
// a ring step that sends before it receives cannot deadlock on socket buffers.
class TcpTransport : public Transport {
 public:
  TcpTransport(int rank, int world);
  ~TcpTransport() override;
  int port() const { return port_; }
  bool Connect(const std::vector<int>& ports, int timeout_ms);
  int rank() const override { return rank_; }
  int world() const override { return world_; }
  bool Send(int to, const void* data, std::size_t bytes) override;
  bool Recv(int from, void* data, std::size_t bytes, int timeout_ms) override;
  void set_error(const std::string& e) { error_ = e; }

 private:
  struct Out {
    int to;
    std::vector<std::uint8_t> frame;
  };
  void SenderLoop();
  int rank_, world_, listen_fd_ = -1, port_ = 0;
  std::vector<int> fds_;
  std::mutex mu_;
  std::condition_variable cv_;
  std::deque<Out> queue_;
  std::atomic<bool> stop_{false}, failed_{false};
  std::thread sender_;
};

// Control-plane rendezvous of a multi-process job on one host: rank 0 listens on `master_port`, every other rank
// reports the ephemeral port of its transport, rank 0 answers with the whole table, and all ranks connect
// (the reference exchanges its ring ports the same way through `Rendezvous::ExchangeBytes`, src/rendezvous.cc:145).
// Returns false with `t->error()` set when a rank does not show up within `timeout_ms`.
bool RendezvousAndConnect(TcpTransport* t, int master_port, int timeout_ms);

// Sum all-reduce of `count` floats in place: reduce-scatter then all-gather around the ring, chunk =
// ceil(count / world), the last chunks may be short or empty. Every rank ends with bit-identical data (each
// chunk is summed in one fixed order, then copied). Returns false when a peer does not answer in `timeout_ms`.
bool RingAllReduceSum(Transport* t, float* data, std::size_t count, int timeout_ms = 60000);

// Control-plane all-gather: every rank contributes `mine`; `out[r]` is rank r's contribution on return.
bool AllGatherBytes(Transport* t, const std::vector<std::uint8_t>& mine, std::vector<std::vector<std::uint8_t>>* out,
                    int timeout_ms = 60000);

}  // namespace ncb
