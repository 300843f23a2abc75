#include "collective.h"

#include <arpa/inet.h>
#include <netinet/in.h>
#include <netinet/tcp.h>
#include <poll.h>
#include <sys/socket.h>
#include <unistd.h>

#include <algorithm>
#include <chrono>
#include <cstring>

namespace ncb {

// ------------------------------------------------------------------------------------------ memory transport
MemoryHub::MemoryHub(int world) : world_(std::max(1, world)) {
  boxes_.resize(static_cast<std::size_t>(world_) * world_);
  for (auto& b : boxes_) b = std::make_unique<Box>();
}

void MemoryHub::DropNext(int from, int to, int count) {
  Box& b = box(from, to);
  std::lock_guard<std::mutex> lock(b.mu);
  b.drop = count;
}

class MemoryTransport : public Transport {
 public:
  MemoryTransport(MemoryHub* hub, int rank) : hub_(hub), rank_(rank) {}
  int rank() const override { return rank_; }
  int world() const override { return hub_->world(); }
  bool Send(int to, const void* data, std::size_t bytes) override {
    if (to < 0 || to >= hub_->world()) return false;
    MemoryHub::Box& b = hub_->box(rank_, to);
    {
      std::lock_guard<std::mutex> lock(b.mu);
      if (b.drop > 0) {
        --b.drop;
        return true;
      }
      const auto* p = static_cast<const std::uint8_t*>(data);
      b.q.emplace_back(p, p + bytes);
    }
    b.cv.notify_one();
    return true;
  }
  bool Recv(int from, void* data, std::size_t bytes, int timeout_ms) override {
    if (from < 0 || from >= hub_->world()) return false;
    MemoryHub::Box& b = hub_->box(from, rank_);
    std::unique_lock<std::mutex> lock(b.mu);
    if (!b.cv.wait_for(lock, std::chrono::milliseconds(timeout_ms), [&] { return !b.q.empty(); })) {
      error_ = "no message from rank " + std::to_string(from) + " within " + std::to_string(timeout_ms) + " ms";
      return false;
    }
    std::vector<std::uint8_t> msg = std::move(b.q.front());
    b.q.pop_front();
    if (msg.size() != bytes) {
      error_ = "message size mismatch from rank " + std::to_string(from);
      return false;
    }
    if (bytes) std::memcpy(data, msg.data(), bytes);
    return true;
  }

 private:
  MemoryHub* hub_;
  int rank_;
};

std::unique_ptr<Transport> MemoryHub::Endpoint(int rank) { return std::make_unique<MemoryTransport>(this, rank); }

// ------------------------------------------------------------------------------------------ TCP transport
namespace {

constexpr std::uint32_t kFrameMagic = 0x4E435446u;  // "NCTF"

struct FrameHeader {
  std::uint32_t magic;
  std::uint32_t sender;
  std::uint64_t bytes;
};
static_assert(sizeof(FrameHeader) == 16, "frame header is 16 bytes");

bool WriteAll(int fd, const void* data, std::size_t bytes) {
  const auto* p = static_cast<const std::uint8_t*>(data);
  while (bytes > 0) {
    const ssize_t n = ::send(fd, p, bytes, MSG_NOSIGNAL);
    if (n <= 0) return false;
    p += n;
    bytes -= static_cast<std::size_t>(n);
  }
  return true;
}

bool ReadAll(int fd, void* data, std::size_t bytes, int timeout_ms) {
  auto* p = static_cast<std::uint8_t*>(data);
  const auto deadline = std::chrono::steady_clock::now() + std::chrono::milliseconds(timeout_ms);
  while (bytes > 0) {
    const auto left = std::chrono::duration_cast<std::chrono::milliseconds>(deadline - std::chrono::steady_clock::now());
    if (left.count() <= 0) return false;
    pollfd pf{fd, POLLIN, 0};
    const int r = ::poll(&pf, 1, static_cast<int>(std::min<long long>(left.count(), 1000)));
    if (r < 0) return false;
    if (r == 0) continue;
    const ssize_t n = ::recv(fd, p, bytes, 0);
    if (n <= 0) return false;
    p += n;
    bytes -= static_cast<std::size_t>(n);
  }
  return true;
}

}  // namespace

TcpTransport::TcpTransport(int rank, int world) : rank_(rank), world_(std::max(1, world)), fds_(world_, -1) {
  listen_fd_ = ::socket(AF_INET, SOCK_STREAM, 0);
  if (listen_fd_ < 0) {
    error_ = "socket() failed";
    return;
  }
  int one = 1;
  ::setsockopt(listen_fd_, SOL_SOCKET, SO_REUSEADDR, &one, sizeof(one));
  sockaddr_in addr{};
  addr.sin_family = AF_INET;
  addr.sin_addr.s_addr = htonl(INADDR_LOOPBACK);
  addr.sin_port = 0;
  if (::bind(listen_fd_, reinterpret_cast<sockaddr*>(&addr), sizeof(addr)) != 0 || ::listen(listen_fd_, world_) != 0) {
    error_ = "bind/listen on 127.0.0.1 failed";
    ::close(listen_fd_);
    listen_fd_ = -1;
    return;
  }
  socklen_t len = sizeof(addr);
  ::getsockname(listen_fd_, reinterpret_cast<sockaddr*>(&addr), &len);
  port_ = ntohs(addr.sin_port);
}

TcpTransport::~TcpTransport() {
  {
    std::lock_guard<std::mutex> lock(mu_);
    stop_ = true;
  }
  cv_.notify_all();
  if (sender_.joinable()) sender_.join();
  for (int fd : fds_)
    if (fd >= 0) ::close(fd);
  if (listen_fd_ >= 0) ::close(listen_fd_);
}

bool TcpTransport::Connect(const std::vector<int>& ports, int timeout_ms) {
  if (listen_fd_ < 0 || static_cast<int>(ports.size()) != world_) return false;
  int one = 1;
  // connect to every higher rank, announce who we are
  for (int peer = rank_ + 1; peer < world_; ++peer) {
    const int fd = ::socket(AF_INET, SOCK_STREAM, 0);
    sockaddr_in addr{};
    addr.sin_family = AF_INET;
    addr.sin_addr.s_addr = htonl(INADDR_LOOPBACK);
    addr.sin_port = htons(static_cast<std::uint16_t>(ports[peer]));
    const auto deadline = std::chrono::steady_clock::now() + std::chrono::milliseconds(timeout_ms);
    bool ok = false;
    while (std::chrono::steady_clock::now() < deadline) {
      if (::connect(fd, reinterpret_cast<sockaddr*>(&addr), sizeof(addr)) == 0) {
        ok = true;
        break;
      }
      std::this_thread::sleep_for(std::chrono::milliseconds(20));
    }
    const std::uint32_t hello = static_cast<std::uint32_t>(rank_);
    if (!ok || !WriteAll(fd, &hello, 4)) {
      error_ = "cannot reach rank " + std::to_string(peer);
      ::close(fd);
      return false;
    }
    ::setsockopt(fd, IPPROTO_TCP, TCP_NODELAY, &one, sizeof(one));
    fds_[peer] = fd;
  }
  // accept one connection from every lower rank
  for (int k = 0; k < rank_; ++k) {
    pollfd pf{listen_fd_, POLLIN, 0};
    if (::poll(&pf, 1, timeout_ms) <= 0) {
      error_ = "a lower rank did not connect";
      return false;
    }
    const int fd = ::accept(listen_fd_, nullptr, nullptr);
    std::uint32_t who = 0;
    if (fd < 0 || !ReadAll(fd, &who, 4, timeout_ms) || who >= static_cast<std::uint32_t>(rank_) || fds_[who] >= 0) {
      error_ = "bad hello on an accepted connection";
      if (fd >= 0) ::close(fd);
      return false;
    }
    ::setsockopt(fd, IPPROTO_TCP, TCP_NODELAY, &one, sizeof(one));
    fds_[who] = fd;
  }
  sender_ = std::thread([this] { SenderLoop(); });
  return true;
}

void TcpTransport::SenderLoop() {
  for (;;) {
    Out out;
    {
      std::unique_lock<std::mutex> lock(mu_);
      cv_.wait(lock, [&] { return stop_ || !queue_.empty(); });
      if (queue_.empty()) return;  // stop requested and drained
      out = std::move(queue_.front());
      queue_.pop_front();
    }
    if (!WriteAll(fds_[out.to], out.frame.data(), out.frame.size())) failed_ = true;
  }
}

bool TcpTransport::Send(int to, const void* data, std::size_t bytes) {
  if (to < 0 || to >= world_ || to == rank_ || fds_[to] < 0 || failed_) return false;
  Out out;
  out.to = to;
  out.frame.resize(sizeof(FrameHeader) + bytes);
  const FrameHeader h{kFrameMagic, static_cast<std::uint32_t>(rank_), static_cast<std::uint64_t>(bytes)};
  std::memcpy(out.frame.data(), &h, sizeof(h));
  if (bytes) std::memcpy(out.frame.data() + sizeof(h), data, bytes);
  {
    std::lock_guard<std::mutex> lock(mu_);
    queue_.push_back(std::move(out));
  }
  cv_.notify_one();
  return true;
}

bool TcpTransport::Recv(int from, void* data, std::size_t bytes, int timeout_ms) {
  if (from < 0 || from >= world_ || from == rank_ || fds_[from] < 0) return false;
  FrameHeader h{};
  if (!ReadAll(fds_[from], &h, sizeof(h), timeout_ms)) {
    error_ = "no frame from rank " + std::to_string(from) + " within " + std::to_string(timeout_ms) + " ms";
    return false;
  }
  if (h.magic != kFrameMagic || h.sender != static_cast<std::uint32_t>(from) || h.bytes != bytes) {
    error_ = "bad frame from rank " + std::to_string(from);
    return false;
  }
  if (bytes && !ReadAll(fds_[from], data, bytes, timeout_ms)) {
    error_ = "short frame from rank " + std::to_string(from);
    return false;
  }
  return true;
}

// ------------------------------------------------------------------------------------------ rendezvous
bool RendezvousAndConnect(TcpTransport* t, int master_port, int timeout_ms) {
  const int world = t->world(), rank = t->rank();
  std::vector<int> ports(world, 0);
  ports[rank] = t->port();
  if (world == 1) return t->Connect(ports, timeout_ms);
  sockaddr_in addr{};
  addr.sin_family = AF_INET;
  addr.sin_addr.s_addr = htonl(INADDR_LOOPBACK);
  addr.sin_port = htons(static_cast<std::uint16_t>(master_port));
  if (rank == 0) {
    const int fd = ::socket(AF_INET, SOCK_STREAM, 0);
    int one = 1;
    ::setsockopt(fd, SOL_SOCKET, SO_REUSEADDR, &one, sizeof(one));
    if (fd < 0 || ::bind(fd, reinterpret_cast<sockaddr*>(&addr), sizeof(addr)) != 0 || ::listen(fd, world) != 0) {
      t->set_error("rendezvous: cannot listen on 127.0.0.1:" + std::to_string(master_port));
      if (fd >= 0) ::close(fd);
      return false;
    }
    std::vector<int> peers;
    bool ok = true;
    for (int k = 1; k < world && ok; ++k) {
      pollfd pf{fd, POLLIN, 0};
      if (::poll(&pf, 1, timeout_ms) <= 0) {
        t->set_error("rendezvous: " + std::to_string(world - k) + " rank(s) did not join");
        ok = false;
        break;
      }
      const int c = ::accept(fd, nullptr, nullptr);
      std::uint32_t hello[2] = {0, 0};
      if (c < 0 || !ReadAll(c, hello, sizeof(hello), timeout_ms) || hello[0] == 0 || hello[0] >= static_cast<std::uint32_t>(world) ||
          ports[hello[0]] != 0) {
        t->set_error("rendezvous: bad hello");
        if (c >= 0) ::close(c);
        ok = false;
        break;
      }
      ports[hello[0]] = static_cast<int>(hello[1]);
      peers.push_back(c);
    }
    std::vector<std::uint32_t> table(ports.begin(), ports.end());
    for (int c : peers) {
      if (ok) ok = WriteAll(c, table.data(), table.size() * 4);
      ::close(c);
    }
    ::close(fd);
    if (!ok) return false;
  } else {
    const int fd = ::socket(AF_INET, SOCK_STREAM, 0);
    const auto deadline = std::chrono::steady_clock::now() + std::chrono::milliseconds(timeout_ms);
    bool connected = false;
    while (std::chrono::steady_clock::now() < deadline) {
      if (::connect(fd, reinterpret_cast<sockaddr*>(&addr), sizeof(addr)) == 0) {
        connected = true;
        break;
      }
      std::this_thread::sleep_for(std::chrono::milliseconds(50));
    }
    const std::uint32_t hello[2] = {static_cast<std::uint32_t>(rank), static_cast<std::uint32_t>(t->port())};
    std::vector<std::uint32_t> table(world);
    const bool ok = connected && WriteAll(fd, hello, sizeof(hello)) && ReadAll(fd, table.data(), table.size() * 4, timeout_ms);
    ::close(fd);
    if (!ok) {
      t->set_error("rendezvous: rank 0 did not answer on 127.0.0.1:" + std::to_string(master_port));
      return false;
    }
    for (int r = 0; r < world; ++r) ports[r] = static_cast<int>(table[r]);
  }
  return t->Connect(ports, timeout_ms);
}

// ------------------------------------------------------------------------------------------ collectives
bool RingAllReduceSum(Transport* t, float* data, std::size_t count, int timeout_ms) {
  const int n = t->world(), r = t->rank();
  if (n <= 1 || count == 0) return true;
  const std::size_t chunk = (count + n - 1) / n;
  auto span = [&](int c, std::size_t* lo, std::size_t* len) {
    *lo = std::min(count, static_cast<std::size_t>(c) * chunk);
    *len = std::min(count, *lo + chunk) - *lo;
  };
  const int next = (r + 1) % n, prev = (r + n - 1) % n;
  std::vector<float> incoming(chunk);
  // reduce-scatter: in step s rank r sends chunk (r - s) and adds what it receives into chunk (r - s - 1); after
  // n-1 steps rank r holds the complete sum of chunk (r + 1)
  for (int s = 0; s < n - 1; ++s) {
    std::size_t slo, slen, rlo, rlen;
    span(((r - s) % n + n) % n, &slo, &slen);
    span(((r - s - 1) % n + n) % n, &rlo, &rlen);
    if (!t->Send(next, data + slo, slen * sizeof(float))) return false;
    if (!t->Recv(prev, incoming.data(), rlen * sizeof(float), timeout_ms)) return false;
    for (std::size_t i = 0; i < rlen; ++i) data[rlo + i] += incoming[i];
  }
  // all-gather: circulate the finished chunks, received straight into place
  for (int s = 0; s < n - 1; ++s) {
    std::size_t slo, slen, rlo, rlen;
    span(((r + 1 - s) % n + n) % n, &slo, &slen);
    span(((r - s) % n + n) % n, &rlo, &rlen);
    if (!t->Send(next, data + slo, slen * sizeof(float))) return false;
    if (!t->Recv(prev, data + rlo, rlen * sizeof(float), timeout_ms)) return false;
  }
  return true;
}

bool AllGatherBytes(Transport* t, const std::vector<std::uint8_t>& mine, std::vector<std::vector<std::uint8_t>>* out,
                    int timeout_ms) {
  const int n = t->world(), r = t->rank();
  out->assign(n, {});
  (*out)[r] = mine;
  for (int peer = 0; peer < n; ++peer) {
    if (peer == r) continue;
    const std::uint64_t len = mine.size();
    if (!t->Send(peer, &len, sizeof(len)) || !t->Send(peer, mine.data(), mine.size())) return false;
  }
  for (int peer = 0; peer < n; ++peer) {
    if (peer == r) continue;
    std::uint64_t len = 0;
    if (!t->Recv(peer, &len, sizeof(len), timeout_ms)) return false;
    (*out)[peer].resize(len);
    if (!t->Recv(peer, (*out)[peer].data(), len, timeout_ms)) return false;
  }
  return true;
}

}  // namespace ncb
