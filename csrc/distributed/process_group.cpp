#include "process_group.h"

#include <cstddef>
#include <cstdlib>
#include <map>
#include <set>

#include <ATen/ATen.h>
#include <c10/util/Exception.h>
#include <cstring>
#include <thread>

#include <poll.h>
#include <sys/socket.h>
#include <sys/un.h>
#include <unistd.h>

#include "../runtime/caching_allocator.h"
#include "../runtime/device.h"
#include "../runtime/log.h"
#include "../runtime/profiler.h"
#include "../runtime/tensor_impl.h"

namespace catch_b200 {

namespace ops {
void note_kernel_launch();
}

namespace {

int dtype_code(at::ScalarType t) {
  switch (t) {
    case at::kFloat: return B200_F32;
    case at::kBFloat16: return B200_BF16;
    case at::kHalf: return B200_F16;
    case at::kDouble: return B200_F64;
    case at::kInt: return B200_I32;
    case at::kLong: return B200_I64;
    default: return -1;
  }
}
int op_code(const c10d::ReduceOp& op) {
  switch (static_cast<c10d::ReduceOp::RedOpType>(op)) {
    case c10d::ReduceOp::SUM: return COMM_SUM;
    case c10d::ReduceOp::PRODUCT: return COMM_PROD;
    case c10d::ReduceOp::MIN: return COMM_MIN;
    case c10d::ReduceOp::MAX: return COMM_MAX;
    case c10d::ReduceOp::AVG: return COMM_AVG;
    default: TORCH_CHECK(false, "bwccl: unsupported reduce op");
  }
}
size_t env_mb(const char* name, size_t dflt) {
  const char* s = std::getenv(name);
  return (s && *s) ? static_cast<size_t>(std::atoll(s)) : dflt;
}
#define COMM_CHECK(expr)                                                                         \
  do {                                                                                           \
    ::catch_b200::ops::note_kernel_launch();                                                     \
    ::catch_b200::KernelTraceScope _trace(#expr);                                                \
    int _e = (expr);                                                                             \
    TORCH_CHECK(_e == 0, "bwccl: device call failed: ", device_error_string(_e), " (", #expr, ")"); \
  } while (0)

std::atomic<int> g_pg_counter{0};
}  // namespace

int next_process_group_id() { return g_pg_counter.fetch_add(1); }

// ------------------------------------------------------------------------ FdExchange
// Passes file descriptors (shareable handles of device memory) between the ranks of one host over
// abstract-namespace Unix sockets with SCM_RIGHTS.  Every rank listens on "\0<token>/<rank>"; a sender
// connects, sends {source rank, tag} with the descriptor attached, and closes.  Connections queue in the
// listener's backlog, so everybody can send first and receive afterwards without a helper thread.
class FdExchange {
 public:
  FdExchange(const std::string& token, int rank) : token_(token), rank_(rank) {
    listen_fd_ = ::socket(AF_UNIX, SOCK_STREAM, 0);
    TORCH_CHECK(listen_fd_ >= 0, "bwccl: cannot create a Unix socket");
    sockaddr_un addr;
    const socklen_t len = fill(addr, rank);
    TORCH_CHECK(::bind(listen_fd_, reinterpret_cast<sockaddr*>(&addr), len) == 0, "bwccl: cannot bind the handle-exchange socket");
    TORCH_CHECK(::listen(listen_fd_, 128) == 0, "bwccl: cannot listen on the handle-exchange socket");
  }
  ~FdExchange() {
    for (auto& kv : stash_) ::close(kv.second);
    if (listen_fd_ >= 0) ::close(listen_fd_);
  }
  void send(int dst, int tag, int fd) {
    const int s = ::socket(AF_UNIX, SOCK_STREAM, 0);
    TORCH_CHECK(s >= 0, "bwccl: cannot create a Unix socket");
    sockaddr_un addr;
    const socklen_t len = fill(addr, dst);
    int rc = -1;
    for (int attempt = 0; attempt < 2000 && rc != 0; ++attempt) {  // the peer may not be listening yet
      rc = ::connect(s, reinterpret_cast<sockaddr*>(&addr), len);
      if (rc != 0) std::this_thread::sleep_for(std::chrono::milliseconds(5));
    }
    TORCH_CHECK(rc == 0, "bwccl: cannot reach rank ", dst, " to hand over a memory handle");
    int payload[2] = {rank_, tag};
    iovec iov{payload, sizeof(payload)};
    char ctrl[CMSG_SPACE(sizeof(int))];
    std::memset(ctrl, 0, sizeof(ctrl));
    msghdr msg{};
    msg.msg_iov = &iov; msg.msg_iovlen = 1;
    msg.msg_control = ctrl; msg.msg_controllen = sizeof(ctrl);
    cmsghdr* c = CMSG_FIRSTHDR(&msg);
    c->cmsg_level = SOL_SOCKET; c->cmsg_type = SCM_RIGHTS; c->cmsg_len = CMSG_LEN(sizeof(int));
    std::memcpy(CMSG_DATA(c), &fd, sizeof(int));
    const ssize_t n = ::sendmsg(s, &msg, 0);
    ::close(s);
    TORCH_CHECK(n == (ssize_t)sizeof(payload), "bwccl: sending a memory handle to rank ", dst, " failed");
  }
  int recv(int src, int tag, std::chrono::milliseconds timeout) {
    const auto key = std::make_pair(src, tag);
    const auto t0 = std::chrono::steady_clock::now();
    for (;;) {
      auto it = stash_.find(key);
      if (it != stash_.end()) {
        const int fd = it->second;
        stash_.erase(it);
        return fd;
      }
      TORCH_CHECK(std::chrono::steady_clock::now() - t0 < timeout, "bwccl: timed out waiting for a memory handle from rank ", src);
      pollfd p{listen_fd_, POLLIN, 0};
      if (::poll(&p, 1, 100) <= 0) continue;
      const int cfd = ::accept(listen_fd_, nullptr, nullptr);
      if (cfd < 0) continue;
      int payload[2] = {-1, -1};
      iovec iov{payload, sizeof(payload)};
      char ctrl[CMSG_SPACE(sizeof(int))];
      msghdr msg{};
      msg.msg_iov = &iov; msg.msg_iovlen = 1;
      msg.msg_control = ctrl; msg.msg_controllen = sizeof(ctrl);
      const ssize_t n = ::recvmsg(cfd, &msg, 0);
      ::close(cfd);
      cmsghdr* c = CMSG_FIRSTHDR(&msg);
      if (n != (ssize_t)sizeof(payload) || !c || c->cmsg_type != SCM_RIGHTS) continue;
      int fd = -1;
      std::memcpy(&fd, CMSG_DATA(c), sizeof(int));
      stash_[std::make_pair(payload[0], payload[1])] = fd;
    }
  }

 private:
  socklen_t fill(sockaddr_un& addr, int rank) const {
    std::memset(&addr, 0, sizeof(addr));
    addr.sun_family = AF_UNIX;
    const std::string name = token_ + "/" + std::to_string(rank);
    TORCH_CHECK(name.size() + 2 < sizeof(addr.sun_path), "bwccl: socket name too long");
    std::memcpy(addr.sun_path + 1, name.data(), name.size());  // leading NUL: abstract namespace
    return static_cast<socklen_t>(offsetof(sockaddr_un, sun_path) + 1 + name.size());
  }
  std::string token_;
  int rank_;
  int listen_fd_ = -1;
  std::map<std::pair<int, int>, int> stash_;
};

// ------------------------------------------------------------------ SymmetricArena
// Layout of one rank's arena: [staging | p2p mailbox | user region | flag block].
// Two ways to make it visible to the peers: cudaMalloc + CUDA IPC handles through the Store (always works),
// or, when every rank's GPU supports NVSwitch multicast and CATCH_B200_NVLS is not 0, a cuMemCreate
// allocation shared as a file descriptor and bound to one multicast object, which adds `mc` (an address
// that reaches the same offset on every rank) for the in-switch reduction kernels.
class SymmetricArena {
 public:
  SymmetricArena(int device, int rank, int world, const c10::intrusive_ptr<c10d::Store>& store, const std::string& uid,
                 std::chrono::milliseconds timeout)
      : device_(device), rank_(rank), world_(world) {
    TORCH_CHECK(world <= B200_COMM_MAX_RANKS, "bwccl: at most ", B200_COMM_MAX_RANKS, " ranks per group");
    staging_ = env_mb("CATCH_B200_SYMM_STAGING_MB", 128) << 20;
    mailbox_ = size_t(16) << 20;
    user_ = env_mb("CATCH_B200_SYMM_USER_MB", 1536) << 20;
    total_ = staging_ + mailbox_ + user_ + B200_COMM_FLAG_BYTES;
    DeviceSwitch sw(device);
    std::memset(&ctx_, 0, sizeof(ctx_));
    ctx_.rank = rank;
    ctx_.world = world;
    auto barrier = [&](const std::string& name) {
      store->add(uid + "/" + name, 1);
      const auto t0 = std::chrono::steady_clock::now();
      while (store->add(uid + "/" + name, 0) < world) {
        TORCH_CHECK(std::chrono::steady_clock::now() - t0 < timeout, "bwccl: timed out waiting for peers (", name, ")");
        std::this_thread::sleep_for(std::chrono::milliseconds(2));
      }
    };
    // every rank votes; the multicast path is taken only if all of them can
    // Default: from four ranks up.  Through the switch every rank sends its whole message once and receives the
    // whole result once (about 1 + 1/world message sizes per direction) against 2 (world - 1) / world for peer
    // loads and stores: a gain of 1.2x at four ranks and 1.56x at eight, but a loss at two (1.5 against 1.0).
    // CATCH_B200_NVLS=1 forces it on for any world size, =0 turns it off.
    int mine = 0;
    const char* env = std::getenv("CATCH_B200_NVLS");
    const bool forced_on = env && std::string(env) == "1", forced_off = env && std::string(env) == "0";
    if (!forced_off && world > 1 && (forced_on || world >= 4)) b200_vmm_multicast_supported(device, &mine);
    store->add(uid + "/vmm_votes", mine);
    barrier("vmm_voted");
    vmm_ = store->add(uid + "/vmm_votes", 0) == world;
    if (vmm_) {
      try {
        setup_vmm(store, uid, timeout, barrier);
      } catch (const std::exception& e) {
        // all ranks run the same steps on the same kind of GPU, so they fail (or not) together
        B200LOG(WARNING) << "bwccl: multicast set-up failed (" << e.what() << "); using CUDA IPC peer mappings only.";
        teardown_vmm();
        vmm_ = false;
      }
      // agree on the outcome: one failing rank sends everybody back to the IPC path
      store->add(uid + "/vmm_ok", vmm_ ? 1 : 0);
      barrier("vmm_done");
      if (store->add(uid + "/vmm_ok", 0) != world && vmm_) {
        teardown_vmm();
        vmm_ = false;
      }
    }
    if (!vmm_) setup_ipc(store, uid, timeout);
    COMM_CHECK(b200_memset_async(static_cast<char*>(base_) + total_ - B200_COMM_FLAG_BYTES, 0, B200_COMM_FLAG_BYTES, nullptr));
    COMM_CHECK(b200_device_synchronize());
    void* host = nullptr;
    void* dev = nullptr;
    COMM_CHECK(b200_host_alloc_mapped(&host, &dev, 64));
    status_host_ = static_cast<int*>(host);
    status_dev_ = static_cast<int*>(dev);
    ctx_.status = status_dev_;
    for (int p = 0; p < world; ++p)
      ctx_.flags[p] = reinterpret_cast<unsigned long long*>(static_cast<char*>(ctx_.arena[p]) + total_ - B200_COMM_FLAG_BYTES);
    // nobody may signal before every rank has zeroed its flags and mapped its peers
    barrier("mapped");
    B200LOG(INFO) << "bwccl arena of rank " << rank << ": " << (total_ >> 20) << " MiB, "
                  << (vmm_ ? "multicast (NVLS) mapping" : "CUDA IPC peer mappings");
  }
  ~SymmetricArena() {
    try {
      DeviceSwitch sw(device_);
      b200_device_synchronize();
      if (vmm_) {
        teardown_vmm();
      } else {
        for (void* p : opened_) b200_ipc_close_handle(p);
        b200_free(base_);
      }
      b200_host_free(status_host_);
    } catch (...) {
    }
  }
  B200CommCtx ctx() const { return ctx_; }
  bool multicast() const { return vmm_ && ctx_.mc != nullptr; }
  char* local() const { return static_cast<char*>(base_); }
  size_t staging_bytes() const { return staging_; }
  size_t mailbox_offset() const { return staging_; }
  size_t mailbox_bytes() const { return mailbox_; }
  size_t user_alloc(size_t bytes) {
    bytes = (bytes + 255) / 256 * 256;
    TORCH_CHECK(user_used_ + bytes <= user_, "bwccl: symmetric user region exhausted (", user_ >> 20,
                " MiB); raise CATCH_B200_SYMM_USER_MB");
    const size_t off = staging_ + mailbox_ + user_used_;
    user_used_ += bytes;
    return off;
  }
  size_t offset_of(const void* p) const {
    const char* c = static_cast<const char*>(p);
    TORCH_CHECK(c >= local() && c < local() + total_, "bwccl: tensor does not live in the symmetric arena");
    return static_cast<size_t>(c - local());
  }
  int* status_host() const { return status_host_; }
  void* counter_ptr() const { return local() + total_ - B200_COMM_FLAG_BYTES + B200_COMM_COUNTER_SLOT * 8; }
  void set_timeout_ns(unsigned long long ns) { ctx_.timeout_ns = ns; }

 private:
  void setup_ipc(const c10::intrusive_ptr<c10d::Store>& store, const std::string& uid, std::chrono::milliseconds timeout) {
    COMM_CHECK(b200_malloc(&base_, total_));
    char handle[64];
    COMM_CHECK(b200_ipc_get_handle(base_, handle));
    store->set(uid + "/ipc/" + std::to_string(rank_), std::vector<uint8_t>(handle, handle + 64));
    for (int p = 0; p < world_; ++p) {
      void* ptr = base_;
      if (p != rank_) {
        const std::string key = uid + "/ipc/" + std::to_string(p);
        store->wait({key}, timeout);
        auto h = store->get(key);
        TORCH_CHECK(h.size() == 64, "bwccl: malformed IPC handle from rank ", p);
        COMM_CHECK(b200_ipc_open_handle(reinterpret_cast<const char*>(h.data()), &ptr));
        opened_.push_back(ptr);
      }
      ctx_.arena[p] = ptr;
    }
  }
  template <typename Barrier>
  void setup_vmm(const c10::intrusive_ptr<c10d::Store>& store, const std::string& uid, std::chrono::milliseconds timeout,
                 Barrier&& barrier) {
    // a token that only this job's ranks know names the sockets
    if (rank_ == 0) {
      const std::string tok = "bwccl-" + std::to_string(::getpid()) + "-" + std::to_string(std::chrono::steady_clock::now().time_since_epoch().count());
      store->set(uid + "/fdtoken", std::vector<uint8_t>(tok.begin(), tok.end()));
    }
    store->wait({uid + "/fdtoken"}, timeout);
    auto tokv = store->get(uid + "/fdtoken");
    FdExchange fdx(std::string(tokv.begin(), tokv.end()), rank_);
    COMM_CHECK(b200_vmm_round_size(device_, world_, total_, &mapped_bytes_));
    int fd = -1;
    COMM_CHECK(b200_vmm_alloc(mapped_bytes_, device_, &base_, &mem_handle_, &fd));
    barrier("fd_listening");  // every rank's socket exists
    for (int p = 0; p < world_; ++p)
      if (p != rank_) fdx.send(p, /*tag=*/0, fd);
    ::close(fd);
    peer_ptr_.assign(world_, nullptr);
    peer_handle_.assign(world_, 0);
    for (int p = 0; p < world_; ++p) {
      if (p == rank_) {
        ctx_.arena[p] = base_;
        continue;
      }
      const int pfd = fdx.recv(p, 0, timeout);
      COMM_CHECK(b200_vmm_import(pfd, mapped_bytes_, device_, &peer_ptr_[p], &peer_handle_[p]));
      ctx_.arena[p] = peer_ptr_[p];
    }
    // one multicast object: created by rank 0, imported by the others, every device added, every allocation bound
    if (rank_ == 0) {
      int mfd = -1;
      COMM_CHECK(b200_mc_create(world_, mapped_bytes_, &mc_handle_, &mfd));
      for (int p = 1; p < world_; ++p) fdx.send(p, /*tag=*/1, mfd);
      ::close(mfd);
    } else {
      const int mfd = fdx.recv(0, 1, timeout);
      COMM_CHECK(b200_mc_import(mfd, &mc_handle_));
    }
    COMM_CHECK(b200_mc_add_device(mc_handle_, device_));
    barrier("mc_added");
    COMM_CHECK(b200_mc_bind(mc_handle_, mem_handle_, mapped_bytes_));
    mc_bound_ = true;
    barrier("mc_bound");
    void* mc_ptr = nullptr;
    COMM_CHECK(b200_mc_map(mc_handle_, mapped_bytes_, device_, &mc_ptr));
    ctx_.mc = mc_ptr;
  }
  void teardown_vmm() {
    if (ctx_.mc || mc_handle_) b200_mc_release(ctx_.mc, mapped_bytes_, mc_handle_, device_, mc_bound_ ? 1 : 0);
    ctx_.mc = nullptr;
    mc_handle_ = 0;
    mc_bound_ = false;
    for (size_t p = 0; p < peer_ptr_.size(); ++p)
      if (peer_ptr_[p]) b200_vmm_release(peer_ptr_[p], mapped_bytes_, peer_handle_[p]);
    peer_ptr_.clear();
    peer_handle_.clear();
    if (base_ && mem_handle_) b200_vmm_release(base_, mapped_bytes_, mem_handle_);
    base_ = nullptr;
    mem_handle_ = 0;
  }

  int device_, rank_, world_;
  void* base_ = nullptr;
  size_t staging_, mailbox_, user_, total_, user_used_ = 0;
  int* status_host_ = nullptr;
  int* status_dev_ = nullptr;
  std::vector<void*> opened_;
  B200CommCtx ctx_;
  // multicast path
  bool vmm_ = false, mc_bound_ = false;
  size_t mapped_bytes_ = 0;
  unsigned long long mem_handle_ = 0, mc_handle_ = 0;
  std::vector<void*> peer_ptr_;
  std::vector<unsigned long long> peer_handle_;
};

// ------------------------------------------------------------------------- WorkB200
WorkB200::WorkB200(int rank, c10d::OpType op, std::vector<at::Tensor> outputs, int device, int* status,
                   std::chrono::milliseconds timeout)
    : c10d::Work(rank, op), outputs_(std::move(outputs)), device_(device), status_(status), timeout_(timeout) {}

void WorkB200::finish_host(std::exception_ptr err) {
  host_done_ = true;
  error_ = err;
}
void WorkB200::check_status() const {
  if (error_) std::rethrow_exception(error_);
  if (status_ && *((volatile int*)status_) != 0) {
    const int s = *((volatile int*)status_);
    TORCH_CHECK_WITH(DistBackendError, false, "bwccl: a device-side wait timed out (status ", s & 0xff, ", waiting for rank ",
                     (s >> 8) & 0xff, "). A peer did not reach the collective in time.");
  }
}
bool WorkB200::isCompleted() { return host_done_ || notifier_.query(); }
bool WorkB200::isSuccess() const { return !error_ && !(status_ && *((volatile int*)status_) != 0); }
std::exception_ptr WorkB200::exception() const {
  try {
    check_status();
  } catch (...) {
    return std::current_exception();
  }
  return nullptr;
}
void WorkB200::synchronize() {
  if (host_done_) {
    check_status();
    return;
  }
  // device-side ordering: later work on the current queue waits for the collective
  notifier_.wait(getCurrentQueue(device_));
  if (flags().blocking_wait) {
    notifier_.synchronize();
    check_status();
  }
}
bool WorkB200::wait(std::chrono::milliseconds timeout) {
  if (host_done_) {
    check_status();
    return true;
  }
  if (timeout == kNoTimeout && !flags().blocking_wait) {
    synchronize();
    return true;
  }
  const auto limit = timeout == kNoTimeout ? timeout_ : timeout;
  const auto t0 = std::chrono::steady_clock::now();
  while (!notifier_.query()) {
    if (std::chrono::steady_clock::now() - t0 > limit) {
      TORCH_CHECK_WITH(DistBackendError, false, "bwccl: collective did not complete within ", limit.count(), " ms");
    }
    std::this_thread::sleep_for(std::chrono::microseconds(50));
  }
  check_status();
  notifier_.wait(getCurrentQueue(device_));
  return true;
}
c10::intrusive_ptr<c10::ivalue::Future> WorkB200::getFuture() {
  if (!future_) {
    future_ = c10::make_intrusive<c10::ivalue::Future>(c10::ListType::create(c10::TensorType::get()));
    // Completion of the future means "ordered on the current queue": consumers of the
    // value run on that queue, which waits on the notifier.
    if (!host_done_) notifier_.wait(getCurrentQueue(device_));
    if (error_) future_->setError(error_);
    else future_->markCompleted(c10::IValue(outputs_));
  }
  return future_;
}

// ------------------------------------------------------------------ ProcessGroupB200
namespace {
std::mutex g_groups_mu;
std::set<ProcessGroupB200*> g_groups;
}  // namespace

ProcessGroupB200::ProcessGroupB200(const c10::intrusive_ptr<c10d::Store>& store, int rank, int size,
                                   std::chrono::milliseconds timeout)
    : c10d::Backend(rank, size), store_(store), timeout_(timeout), send_seq_(size, 0), recv_seq_(size, 0) {
  uid_ = "bwccl/" + std::to_string(next_process_group_id());
  B200LOG(INFO) << "ProcessGroupB200 rank " << rank << "/" << size << " uid " << uid_;
  if (const char* e = std::getenv("CATCH_B200_HEARTBEAT_MS")) hb_interval_ms_ = std::atoll(e);
  if (const char* e = std::getenv("CATCH_B200_HEARTBEAT_TIMEOUT_MS")) hb_timeout_ms_ = std::atoll(e);
  {
    std::lock_guard<std::mutex> lk(g_groups_mu);
    g_groups.insert(this);
  }
  if (size > 1 && hb_interval_ms_ > 0) start_watchdog();
}

void ProcessGroupB200::start_watchdog() {
  watchdog_ = std::thread([this] {
    try {
      watchdog_loop();
    } catch (const std::exception& e) {
      B200LOG(INFO) << "bwccl watchdog of rank " << rank_ << " stopped: " << e.what();
    } catch (...) {
    }
  });
}

void ProcessGroupB200::watchdog_loop() {
  using clock = std::chrono::steady_clock;
  auto hb_key = [&](int r) { return uid_ + "/hb/" + std::to_string(r); };
  auto bye_key = [&](int r) { return uid_ + "/bye/" + std::to_string(r); };
  std::vector<int64_t> last(size_, -1);
  std::vector<clock::time_point> changed(size_, clock::now());
  std::vector<bool> gone(size_, false);
  for (;;) {
    {
      std::unique_lock<std::mutex> lk(wd_mu_);
      if (wd_cv_.wait_for(lk, std::chrono::milliseconds(hb_interval_ms_), [this] { return wd_stop_; })) break;
    }
    store_->add(hb_key(rank_), 1);
    const auto now = clock::now();
    for (int r = 0; r < size_; ++r) {
      if (r == rank_ || gone[r]) continue;
      const int64_t v = store_->add(hb_key(r), 0);
      if (v != last[r]) {
        last[r] = v;
        changed[r] = now;
        continue;
      }
      if (now - changed[r] < std::chrono::milliseconds(hb_timeout_ms_)) continue;
      if (store_->add(bye_key(r), 0) > 0) {  // it finished and said so
        gone[r] = true;
        continue;
      }
      int64_t expect = -1;
      if (dead_peer_.compare_exchange_strong(expect, r))
        B200LOG(ERROR) << "bwccl: rank " << r << " has sent no heartbeat for " << hb_timeout_ms_ << " ms (seen from rank " << rank_
                       << "); further collectives of this group raise.";
    }
    if (arena_ && !status_logged_.load()) {
      const int s = *((volatile int*)arena_->status_host());
      if (s != 0) {
        status_logged_.store(true);
        B200LOG(ERROR) << "bwccl: a device-side wait of rank " << rank_ << " ran out waiting for rank " << ((s >> 8) & 0xff)
                       << " (status word " << s << ").";
      }
    }
  }
}

void stop_all_watchdogs() {
  std::vector<ProcessGroupB200*> groups;
  {
    std::lock_guard<std::mutex> lk(g_groups_mu);
    groups.assign(g_groups.begin(), g_groups.end());
  }
  for (auto* g : groups) g->stop_watchdog();
}

void ProcessGroupB200::stop_watchdog() {
  if (!watchdog_.joinable()) return;
  {
    std::lock_guard<std::mutex> lk(wd_mu_);
    wd_stop_ = true;
  }
  wd_cv_.notify_all();
  watchdog_.join();
  try {
    store_->add(uid_ + "/bye/" + std::to_string(rank_), 1);
  } catch (...) {
  }
}

ProcessGroupB200::~ProcessGroupB200() {
  stop_watchdog();
  if (hostsim() && size_ > 1) {
    // Under host simulation every message travels through the Store, which usually lives in rank 0's process: rank 0
    // may only go away once the other ranks are done with their last exchange (they can still be reading rank 0's
    // message of a final barrier when rank 0 has already read theirs).
    try {
      const std::string key = uid_ + "/closed";
      store_->add(key, 1);
      if (rank_ == 0) {
        const auto limit = std::min<std::chrono::milliseconds>(timeout_, std::chrono::milliseconds(10000));
        const auto t0 = std::chrono::steady_clock::now();
        while (store_->add(key, 0) < size_ && std::chrono::steady_clock::now() - t0 < limit)
          std::this_thread::sleep_for(std::chrono::milliseconds(2));
      }
    } catch (...) {
    }
  }
  {
    std::lock_guard<std::mutex> lk(g_groups_mu);
    g_groups.erase(this);
  }
  try {
    if (arena_) {
      comm_q_.synchronize();
      send_q_.synchronize();
      recv_q_.synchronize();
    }
  } catch (...) {
  }
}

void ProcessGroupB200::ensure_arena(int device) {
  if (hostsim()) {
    device_ = device;
    return;
  }
  if (arena_) {
    TORCH_CHECK(device == device_, "bwccl: one device per process; this group is bound to device ", device_);
    return;
  }
  device_ = device;
  DeviceSwitch sw(device);
  arena_ = std::make_unique<SymmetricArena>(device, rank_, size_, store_, uid_, timeout_);
  apply_wait_limit();
  comm_q_ = getQueueFromPool(device);
  send_q_ = getQueueFromPool(device);
  recv_q_ = getQueueFromPool(device);
}

void ProcessGroupB200::check_single(const std::vector<at::Tensor>& tensors) const {
  TORCH_CHECK(tensors.size() == 1, "bwccl: expecting one tensor only but got multiple (one device per process)");
  TORCH_CHECK(is_b200(tensors[0]), "bwccl: tensors must live on the blackwell device, got ", tensors[0].device());
  TORCH_CHECK(!tensors[0].is_sparse(), "bwccl: sparse tensors are not supported");
}

void ProcessGroupB200::throw_if_failed() const {
  const int64_t dead = dead_peer_.load();
  TORCH_CHECK_WITH(DistBackendError, dead < 0, "bwccl: rank ", dead, " stopped sending heartbeats (it left or died); ",
                   "nothing was launched.");
  if (arena_ && *((volatile int*)arena_->status_host()) != 0) {
    const int s = *((volatile int*)arena_->status_host());
    TORCH_CHECK_WITH(DistBackendError, false, "bwccl: a previous collective failed (device wait timed out waiting for rank ",
                     (s >> 8) & 0xff, "); the communicator is unusable until clear_status().");
  }
}

c10::intrusive_ptr<WorkB200> ProcessGroupB200::make_work(c10d::OpType op, std::vector<at::Tensor> outputs) {
  return c10::make_intrusive<WorkB200>(rank_, op, std::move(outputs), device_, arena_ ? arena_->status_host() : nullptr,
                                       timeout_);
}

template <typename F>
c10::intrusive_ptr<c10d::Work> ProcessGroupB200::run_on_comm(c10d::OpType op, std::vector<at::Tensor> tensors, F&& fn,
                                                             Queue* q) {
  throw_if_failed();
  DeviceSwitch sw(device_);
  Queue& cq = q ? *q : comm_q_;
  // order the comm queue after everything submitted to the compute queue so far
  Notifier ready(false);
  ready.place(getCurrentQueue(device_));
  ready.wait(cq);
  for (auto& t : tensors) recordQueue(t.storage().data_ptr(), cq);
  auto work = make_work(op, tensors);
  work->keep_alive_ = tensors;
  fn(cq.handle());
  work->notifier_.place(cq);
  if (flags().async_disable) work->notifier_.synchronize();
  return work;
}

// ---- host-simulated transport ----------------------------------------------------------
std::vector<std::vector<uint8_t>> ProcessGroupB200::store_exchange(const std::vector<uint8_t>& mine, bool everyone_sends,
                                                                   int root) {
  // The Store refuses values above 8 MiB: a message is one head key (a flag byte, then either the payload itself or
  // the number of parts) plus, for large messages, part keys of at most kPart bytes each.
  constexpr size_t kPart = 4u << 20;
  const uint64_t s = ++host_seq_;
  auto key = [&](uint64_t seq, int r) { return uid_ + "/x/" + std::to_string(seq) + "/" + std::to_string(r); };
  auto part = [&](uint64_t seq, int r, int i) { return key(seq, r) + "/p" + std::to_string(i); };
  auto ack = [&](uint64_t seq, int r) { return uid_ + "/xa/" + std::to_string(seq) + "/" + std::to_string(r); };
  const bool i_send = everyone_sends || rank_ == root;
  if (i_send) {
    int nparts = 0;
    std::vector<uint8_t> head;
    if (mine.size() <= kPart) {
      head.reserve(mine.size() + 1);
      head.push_back(0);
      head.insert(head.end(), mine.begin(), mine.end());
    } else {
      nparts = static_cast<int>((mine.size() + kPart - 1) / kPart);
      for (int i = 0; i < nparts; ++i) {  // the parts first: a reader that sees the head finds them all
        const size_t b = static_cast<size_t>(i) * kPart, e = std::min(mine.size(), b + kPart);
        store_->set(part(s, rank_, i), std::vector<uint8_t>(mine.begin() + b, mine.begin() + e));
      }
      head.resize(1 + sizeof(uint64_t));
      head[0] = 1;
      const uint64_t n64 = static_cast<uint64_t>(nparts);
      std::memcpy(head.data() + 1, &n64, sizeof(n64));
    }
    store_->set(key(s, rank_), head);
    posted_.emplace_back(s, nparts);
  }
  std::vector<std::vector<uint8_t>> all(size_);
  for (int r = 0; r < size_; ++r) {
    if (!everyone_sends && r != root) continue;
    if (r == rank_) {
      all[r] = mine;
      continue;
    }
    store_->wait({key(s, r)}, timeout_);  // throws on timeout: a missing peer is detected here
    std::vector<uint8_t> head = store_->get(key(s, r));
    TORCH_CHECK(!head.empty(), "bwccl(hostsim): empty message head");
    if (head[0] == 0) {
      all[r].assign(head.begin() + 1, head.end());
    } else {
      uint64_t n64 = 0;
      TORCH_CHECK(head.size() == 1 + sizeof(n64), "bwccl(hostsim): malformed message head");
      std::memcpy(&n64, head.data() + 1, sizeof(n64));
      for (uint64_t i = 0; i < n64; ++i) {
        std::vector<uint8_t> piece = store_->get(part(s, r, static_cast<int>(i)));
        all[r].insert(all[r].end(), piece.begin(), piece.end());
      }
    }
    try {
      store_->add(ack(s, r), 1);          // tell the sender that this reader is done with the message
    } catch (...) {                       // housekeeping only: the data is here (the sender's process may be gone)
    }
  }
  // A posted message is deleted once every other rank has acknowledged it.  (Counting rounds is not
  // enough: the root of a broadcast waits for nobody, so it can be several rounds ahead of a reader.)
  try {
    while (!posted_.empty()) {
      const auto [old, nparts] = posted_.front();
      if (store_->add(ack(old, rank_), 0) < size_ - 1) break;
      for (int i = 0; i < nparts; ++i) store_->deleteKey(part(old, rank_, i));
      store_->deleteKey(key(old, rank_));
      store_->deleteKey(ack(old, rank_));
      posted_.pop_front();
    }
  } catch (...) {  // housekeeping only; a Store that is really gone fails the next exchange
  }
  return all;
}

c10::intrusive_ptr<c10d::Work> ProcessGroupB200::hostsim_collective(c10d::OpType op, std::vector<at::Tensor> outs,
                                                                    std::function<void()> fn) {
  throw_if_failed();
  auto work = c10::make_intrusive<WorkB200>(rank_, op, std::move(outs), device_, nullptr, timeout_);
  try {
    fn();
    work->finish_host();
  } catch (...) {
    work->finish_host(std::current_exception());
    throw;
  }
  return work;
}

static std::vector<uint8_t> to_bytes(const at::Tensor& t) {
  at::Tensor c = t.cpu().contiguous();
  const uint8_t* p = static_cast<const uint8_t*>(c.data_ptr());
  return std::vector<uint8_t>(p, p + c.nbytes());
}
static at::Tensor from_bytes(const std::vector<uint8_t>& b, const at::Tensor& like) {
  at::Tensor c = at::empty(like.sizes(), like.options().device(at::kCPU));
  TORCH_CHECK(b.size() == c.nbytes(), "bwccl(hostsim): message size mismatch (", b.size(), " vs ", c.nbytes(), ")");
  std::memcpy(c.data_ptr(), b.data(), b.size());
  return c;
}
static at::Tensor cpu_reduce(std::vector<at::Tensor>& parts, int op, int world) {
  at::Tensor acc = parts[0].clone();
  for (size_t i = 1; i < parts.size(); ++i) {
    switch (op) {
      case COMM_PROD: acc.mul_(parts[i]); break;
      case COMM_MIN: acc = at::minimum(acc, parts[i]); break;
      case COMM_MAX: acc = at::maximum(acc, parts[i]); break;
      default: acc.add_(parts[i]);
    }
  }
  if (op == COMM_AVG) acc = at::div(acc, world);
  return acc;
}

// ---- collectives -------------------------------------------------------------------------
static at::Tensor arithmetic_view(const at::Tensor& t) {
  // dtypes the kernels cannot add are widened to int32 for the reduction
  if (dtype_code(t.scalar_type()) >= 0) return t.contiguous();
  TORCH_CHECK(c10::isIntegralType(t.scalar_type(), /*includeBool=*/true), "bwccl: unsupported dtype ", t.scalar_type());
  return t.to(at::kInt).contiguous();
}

c10::intrusive_ptr<c10d::Work> ProcessGroupB200::allreduce(std::vector<at::Tensor>& tensors,
                                                           const c10d::AllreduceOptions& opts) {
  check_single(tensors);
  at::Tensor& t = tensors[0];
  ensure_arena(t.device().index());
  const int op = op_code(opts.reduceOp);
  if (hostsim()) {
    return hostsim_collective(c10d::OpType::ALLREDUCE, {t}, [&] {
      auto all = store_exchange(to_bytes(t), true, 0);
      std::vector<at::Tensor> parts;
      for (auto& b : all) parts.push_back(from_bytes(b, t));
      t.copy_(cpu_reduce(parts, op, size_));
    });
  }
  at::Tensor work_t = arithmetic_view(t);
  const bool copy_back = !work_t.is_same(t);
  return run_on_comm(c10d::OpType::ALLREDUCE, {t, work_t}, [&, work_t, copy_back](void* stream) mutable {
    const B200CommCtx ctx = arena_->ctx();
    const size_t es = work_t.element_size();
    const int64_t max_elems = static_cast<int64_t>(arena_->staging_bytes() / es);
    char* p = static_cast<char*>(work_t.data_ptr());
    for (int64_t done = 0; done < work_t.numel(); done += max_elems) {
      const int64_t n = std::min<int64_t>(max_elems, work_t.numel() - done);
      COMM_CHECK(b200_comm_copy(arena_->local(), p + done * es, n * es, stream));
      COMM_CHECK(b200_comm_allreduce(&ctx, 0, n, dtype_code(work_t.scalar_type()), op, 1.0f, ++seq_, 0, stream));
      COMM_CHECK(b200_comm_copy(p + done * es, arena_->local(), n * es, stream));
    }
    if (copy_back) {
      QueueGuard g(comm_q_);
      t.copy_(work_t);
    }
  });
}

c10::intrusive_ptr<c10d::Work> ProcessGroupB200::allreduce_coalesced(std::vector<at::Tensor>& tensors,
                                                                     const c10d::AllreduceCoalescedOptions& opts) {
  c10::intrusive_ptr<c10d::Work> last;
  for (auto& t : tensors) {
    std::vector<at::Tensor> one{t};
    last = allreduce(one, opts);
  }
  return last;
}

c10::intrusive_ptr<c10d::Work> ProcessGroupB200::allreduce_symm(const at::Tensor& t, int64_t op, double scale,
                                                                bool test_no_signal) {
  TORCH_CHECK(!hostsim() && arena_, "allreduce_symm needs the CUDA backend and an initialised arena");
  const size_t off = arena_->offset_of(t.data_ptr());
  return run_on_comm(c10d::OpType::ALLREDUCE, {t}, [&, off](void* stream) {
    const B200CommCtx ctx = arena_->ctx();
    COMM_CHECK(b200_comm_allreduce(&ctx, off, t.numel(), dtype_code(t.scalar_type()), (int)op, (float)scale, ++seq_,
                                   test_no_signal ? 1 : 0, stream));
  });
}

c10::intrusive_ptr<c10d::Work> ProcessGroupB200::broadcast(std::vector<at::Tensor>& tensors,
                                                           const c10d::BroadcastOptions& opts) {
  check_single(tensors);
  at::Tensor& t = tensors[0];
  ensure_arena(t.device().index());
  const int root = static_cast<int>(opts.rootRank);
  if (hostsim()) {
    return hostsim_collective(c10d::OpType::BROADCAST, {t}, [&] {
      auto all = store_exchange(rank_ == root ? to_bytes(t) : std::vector<uint8_t>(), false, root);
      if (rank_ != root) t.copy_(from_bytes(all[root], t));
    });
  }
  at::Tensor c = t.contiguous();
  const bool copy_back = !c.is_same(t);
  return run_on_comm(c10d::OpType::BROADCAST, {t, c}, [&, c, copy_back](void* stream) mutable {
    const B200CommCtx ctx = arena_->ctx();
    const size_t cap = arena_->staging_bytes();
    char* p = static_cast<char*>(c.data_ptr());
    for (size_t done = 0; done < c.nbytes() || done == 0; done += cap) {
      const size_t n = std::min(cap, c.nbytes() - done);
      const uint64_t s = ++seq_;
      if (rank_ == root) {
        COMM_CHECK(b200_comm_copy(arena_->local(), p + done, n, stream));
        COMM_CHECK(b200_comm_signal(&ctx, 0, -1, s, stream));   // data is ready
        COMM_CHECK(b200_comm_signal(&ctx, 1, root, s, stream));  // the root itself has nothing to pull
        COMM_CHECK(b200_comm_wait(&ctx, 1, -1, s, stream));      // every peer has pulled
      } else {
        COMM_CHECK(b200_comm_wait(&ctx, 0, root, s, stream));
        COMM_CHECK(b200_comm_copy(p + done, ctx.arena[root], n, stream));
        COMM_CHECK(b200_comm_signal(&ctx, 1, root, s, stream));
      }
      if (c.nbytes() == 0) break;
    }
    if (copy_back && rank_ != root) {
      QueueGuard g(comm_q_);
      t.copy_(c);
    }
  });
}

c10::intrusive_ptr<c10d::Work> ProcessGroupB200::reduce(std::vector<at::Tensor>& tensors, const c10d::ReduceOptions& opts) {
  check_single(tensors);
  at::Tensor& t = tensors[0];
  ensure_arena(t.device().index());
  const int op = op_code(opts.reduceOp);
  const int root = static_cast<int>(opts.rootRank);
  if (hostsim()) {
    return hostsim_collective(c10d::OpType::REDUCE, {t}, [&] {
      auto all = store_exchange(to_bytes(t), true, 0);
      if (rank_ == root) {
        std::vector<at::Tensor> parts;
        for (auto& b : all) parts.push_back(from_bytes(b, t));
        t.copy_(cpu_reduce(parts, op, size_));
      }
    });
  }
  at::Tensor work_t = arithmetic_view(t);
  // Every rank stages its message in its arena; only the root pulls and combines (peers move no result
  // bytes at all, they just take part in the two barriers of the kernel).
  return run_on_comm(c10d::OpType::REDUCE, {t, work_t}, [&, work_t](void* stream) mutable {
    const B200CommCtx ctx = arena_->ctx();
    const size_t es = work_t.element_size();
    const int64_t max_elems = static_cast<int64_t>(arena_->staging_bytes() / es);
    char* p = static_cast<char*>(work_t.data_ptr());
    for (int64_t done = 0; done < work_t.numel(); done += max_elems) {
      const int64_t n = std::min<int64_t>(max_elems, work_t.numel() - done);
      COMM_CHECK(b200_comm_copy(arena_->local(), p + done * es, n * es, stream));
      COMM_CHECK(b200_comm_reduce_range(&ctx, 0, 0, rank_ == root ? n : 0, p + done * es, dtype_code(work_t.scalar_type()), op,
                                        ++seq_, stream));
    }
    if (rank_ == root && !work_t.is_same(t)) {
      QueueGuard g(comm_q_);
      t.copy_(work_t);
    }
  });
}

// Stages `in` in this rank's arena and pulls every peer's message straight into dsts[peer] (device pointers
// of `bytes` each): no flat temporary, no second copy.
void ProcessGroupB200::gather_into(const at::Tensor& in, const std::vector<char*>& dsts, void* stream) {
  const B200CommCtx ctx = arena_->ctx();
  const size_t cap = arena_->staging_bytes();
  const size_t total = in.nbytes();
  char* src = static_cast<char*>(in.data_ptr());
  for (size_t done = 0; done < total; done += cap) {
    const size_t n = std::min(cap, total - done);
    const uint64_t s = ++seq_;
    COMM_CHECK(b200_comm_copy(arena_->local(), src + done, n, stream));
    COMM_CHECK(b200_comm_signal(&ctx, 0, -1, s, stream));
    COMM_CHECK(b200_comm_wait(&ctx, 0, -1, s, stream));
    for (int i = 0; i < size_; ++i) {
      const int p = (rank_ + i) % size_;
      COMM_CHECK(b200_comm_copy(dsts[p] + done, ctx.arena[p], n, stream));
    }
    COMM_CHECK(b200_comm_signal(&ctx, 1, -1, s, stream));
    COMM_CHECK(b200_comm_wait(&ctx, 1, -1, s, stream));
  }
}

c10::intrusive_ptr<c10d::Work> ProcessGroupB200::_allgather_base(at::Tensor& output, at::Tensor& input,
                                                                 const c10d::AllgatherOptions&) {
  TORCH_CHECK(is_b200(input) && is_b200(output), "bwccl: tensors must live on the blackwell device");
  TORCH_CHECK(output.numel() == input.numel() * size_ && output.scalar_type() == input.scalar_type(),
              "bwccl: all_gather output must hold world_size inputs");
  ensure_arena(input.device().index());
  if (hostsim()) {
    return hostsim_collective(c10d::OpType::_ALLGATHER_BASE, {output}, [&] {
      auto all = store_exchange(to_bytes(input), true, 0);
      at::Tensor flat = output.view({size_, -1});
      for (int r = 0; r < size_; ++r) flat[r].copy_(from_bytes(all[r], input).view({-1}));
    });
  }
  TORCH_CHECK(output.is_contiguous(), "bwccl: all_gather output must be contiguous");
  at::Tensor in = input.contiguous();
  return run_on_comm(c10d::OpType::_ALLGATHER_BASE, {output, in}, [&, in](void* stream) mutable {
    std::vector<char*> dsts(size_);
    for (int r = 0; r < size_; ++r) dsts[r] = static_cast<char*>(output.data_ptr()) + (size_t)r * in.nbytes();
    gather_into(in, dsts, stream);
  });
}

c10::intrusive_ptr<c10d::Work> ProcessGroupB200::allgather(std::vector<std::vector<at::Tensor>>& outputs,
                                                           std::vector<at::Tensor>& inputs,
                                                           const c10d::AllgatherOptions& opts) {
  check_single(inputs);
  TORCH_CHECK(outputs.size() == 1 && static_cast<int>(outputs[0].size()) == size_,
              "bwccl: all_gather expects one output list with world_size tensors");
  at::Tensor& in = inputs[0];
  for (auto& o : outputs[0])
    TORCH_CHECK(o.sizes() == in.sizes() && o.scalar_type() == in.scalar_type(), "bwccl: all_gather output shape / dtype mismatch");
  ensure_arena(in.device().index());
  if (hostsim()) {
    return hostsim_collective(c10d::OpType::ALLGATHER, outputs[0], [&] {
      auto all = store_exchange(to_bytes(in), true, 0);
      for (int r = 0; r < size_; ++r) outputs[0][r].copy_(from_bytes(all[r], in));
    });
  }
  // Contiguous outputs receive the peers' bytes directly; a strided output goes through a dense temporary.
  at::Tensor src = in.contiguous();
  std::vector<at::Tensor> dense(size_);
  std::vector<at::Tensor> used{src};
  for (int r = 0; r < size_; ++r) {
    at::Tensor& o = outputs[0][r];
    dense[r] = o.is_contiguous() ? o : at::empty_like(o, at::MemoryFormat::Contiguous);
    used.push_back(o);
    if (!dense[r].is_same(o)) used.push_back(dense[r]);
  }
  return run_on_comm(c10d::OpType::ALLGATHER, used, [&, src, dense](void* stream) mutable {
    std::vector<char*> dsts(size_);
    for (int r = 0; r < size_; ++r) dsts[r] = static_cast<char*>(dense[r].data_ptr());
    gather_into(src, dsts, stream);
    QueueGuard g(comm_q_);
    for (int r = 0; r < size_; ++r)
      if (!dense[r].is_same(outputs[0][r])) outputs[0][r].copy_(dense[r]);
  });
}

c10::intrusive_ptr<c10d::Work> ProcessGroupB200::_reduce_scatter_base(at::Tensor& output, at::Tensor& input,
                                                                      const c10d::ReduceScatterOptions& opts) {
  TORCH_CHECK(is_b200(input) && is_b200(output), "bwccl: tensors must live on the blackwell device");
  TORCH_CHECK(input.numel() == output.numel() * size_ && input.scalar_type() == output.scalar_type(),
              "bwccl: reduce_scatter input must hold world_size outputs");
  ensure_arena(input.device().index());
  const int op = op_code(opts.reduceOp);
  if (hostsim()) {
    return hostsim_collective(c10d::OpType::_REDUCE_SCATTER_BASE, {output}, [&] {
      auto all = store_exchange(to_bytes(input), true, 0);
      std::vector<at::Tensor> parts;
      for (auto& b : all) parts.push_back(from_bytes(b, input));
      at::Tensor red = cpu_reduce(parts, op, size_);
      output.copy_(red.view({size_, -1})[rank_].view(output.sizes()));
    });
  }
  // Each rank stages its whole input and reduces only its own piece, pulling that piece from every peer:
  // (world - 1) / world of one message crosses NVLink per rank instead of a full all-reduce.
  at::Tensor in = arithmetic_view(input);
  at::Tensor out = (output.is_contiguous() && dtype_code(output.scalar_type()) >= 0)
                       ? output : at::empty(output.sizes(), in.options());
  const int64_t piece = output.numel();
  return run_on_comm(c10d::OpType::_REDUCE_SCATTER_BASE, {output, in, out}, [&, in, out, piece](void* stream) mutable {
    const B200CommCtx ctx = arena_->ctx();
    const size_t es = in.element_size();
    // chunk the pieces so that world * chunk elements fit the staging window
    int64_t max_chunk = std::max<int64_t>(1, static_cast<int64_t>(arena_->staging_bytes() / es) / size_);
    if (max_chunk > 16) max_chunk = max_chunk / 16 * 16;  // slots stay 16-byte aligned
    char* src = static_cast<char*>(in.data_ptr());
    char* dst = static_cast<char*>(out.data_ptr());
    for (int64_t done = 0; done < piece || done == 0; done += max_chunk) {
      const int64_t n = std::min<int64_t>(max_chunk, piece - done);
      for (int r = 0; r < size_; ++r)  // staging layout: [rank 0's chunk | rank 1's chunk | ...], 16-byte aligned slots
        COMM_CHECK(b200_comm_copy(arena_->local() + (size_t)r * max_chunk * es, src + ((size_t)r * piece + done) * es, n * es, stream));
      COMM_CHECK(b200_comm_reduce_range(&ctx, (size_t)rank_ * max_chunk * es, 0, n, dst + done * es, dtype_code(in.scalar_type()), op,
                                        ++seq_, stream));
      if (piece == 0) break;
    }
    if (!out.is_same(output)) {
      QueueGuard g(comm_q_);
      output.copy_(out);
    }
  });
}

c10::intrusive_ptr<c10d::Work> ProcessGroupB200::reduce_scatter(std::vector<at::Tensor>& outputs,
                                                                std::vector<std::vector<at::Tensor>>& inputs,
                                                                const c10d::ReduceScatterOptions& opts) {
  check_single(outputs);
  TORCH_CHECK(inputs.size() == 1 && static_cast<int>(inputs[0].size()) == size_, "bwccl: reduce_scatter expects world_size inputs");
  std::vector<at::Tensor> flat_parts;
  for (auto& t : inputs[0]) flat_parts.push_back(t.reshape({-1}));
  at::Tensor flat = at::cat(flat_parts);
  return _reduce_scatter_base(outputs[0], flat, opts);
}

c10::intrusive_ptr<c10d::Work> ProcessGroupB200::send(std::vector<at::Tensor>& tensors, int dst, int) {
  check_single(tensors);
  TORCH_CHECK(dst != rank_ && dst >= 0 && dst < size_, "bwccl: invalid destination rank ", dst, " (sending to self is not supported)");
  at::Tensor t = tensors[0].contiguous();
  ensure_arena(t.device().index());
  if (hostsim()) {
    return hostsim_collective(c10d::OpType::SEND, {}, [&] {
      const uint64_t s = ++send_seq_[dst];
      store_->set(uid_ + "/p2p/" + std::to_string(rank_) + ">" + std::to_string(dst) + "/" + std::to_string(s), to_bytes(t));
    });
  }
  return run_on_comm(c10d::OpType::SEND, {t}, [&, t](void* stream) mutable {
    const B200CommCtx ctx = arena_->ctx();
    const size_t cap = arena_->mailbox_bytes();
    char* p = static_cast<char*>(t.data_ptr());
    for (size_t done = 0; done < t.nbytes() || done == 0; done += cap) {
      const size_t n = std::min(cap, t.nbytes() - done);
      const uint64_t s = ++send_seq_[dst];
      COMM_CHECK(b200_comm_copy(arena_->local() + arena_->mailbox_offset(), p + done, n, stream));
      COMM_CHECK(b200_comm_signal(&ctx, 2, dst, s, stream));
      COMM_CHECK(b200_comm_wait(&ctx, 3, dst, s, stream));
      if (t.nbytes() == 0) break;
    }
  }, &send_q_);
}

c10::intrusive_ptr<c10d::Work> ProcessGroupB200::recv(std::vector<at::Tensor>& tensors, int src, int) {
  check_single(tensors);
  TORCH_CHECK(src != rank_ && src >= 0 && src < size_, "bwccl: invalid source rank ", src);
  at::Tensor& t = tensors[0];
  ensure_arena(t.device().index());
  if (hostsim()) {
    return hostsim_collective(c10d::OpType::RECV, {t}, [&] {
      const uint64_t s = ++recv_seq_[src];
      const std::string key = uid_ + "/p2p/" + std::to_string(src) + ">" + std::to_string(rank_) + "/" + std::to_string(s);
      store_->wait({key}, timeout_);
      t.copy_(from_bytes(store_->get(key), t));
      store_->deleteKey(key);
    });
  }
  at::Tensor c = t.is_contiguous() ? t : at::empty_like(t, at::MemoryFormat::Contiguous);
  return run_on_comm(c10d::OpType::RECV, {t, c}, [&, c](void* stream) mutable {
    const B200CommCtx ctx = arena_->ctx();
    const size_t cap = arena_->mailbox_bytes();
    char* p = static_cast<char*>(c.data_ptr());
    for (size_t done = 0; done < c.nbytes() || done == 0; done += cap) {
      const size_t n = std::min(cap, c.nbytes() - done);
      const uint64_t s = ++recv_seq_[src];
      COMM_CHECK(b200_comm_wait(&ctx, 2, src, s, stream));
      COMM_CHECK(b200_comm_copy(p + done, static_cast<char*>(ctx.arena[src]) + arena_->mailbox_offset(), n, stream));
      COMM_CHECK(b200_comm_signal(&ctx, 3, src, s, stream));
      if (c.nbytes() == 0) break;
    }
    if (!c.is_same(t)) {
      QueueGuard g(recv_q_);
      t.copy_(c);
    }
  }, &recv_q_);
}

c10::intrusive_ptr<c10d::Work> ProcessGroupB200::barrier(const c10d::BarrierOptions&) {
  ensure_arena(device_ >= 0 ? device_ : current_device());
  if (hostsim()) {
    return hostsim_collective(c10d::OpType::BARRIER, {}, [&] { store_exchange({1}, true, 0); });
  }
  auto work = run_on_comm(c10d::OpType::BARRIER, {}, [&](void* stream) {
    const B200CommCtx ctx = arena_->ctx();
    const uint64_t s = ++seq_;
    COMM_CHECK(b200_comm_signal(&ctx, 0, -1, s, stream));
    COMM_CHECK(b200_comm_wait(&ctx, 0, -1, s, stream));
    COMM_CHECK(b200_comm_signal(&ctx, 1, -1, s, stream));
    COMM_CHECK(b200_comm_wait(&ctx, 1, -1, s, stream));
  });
  // a barrier is a host-visible synchronisation point
  auto w = c10::static_intrusive_pointer_cast<WorkB200>(work);
  w->notifier_.synchronize();
  if (w->exception()) std::rethrow_exception(w->exception());
  return work;
}

c10::intrusive_ptr<c10d::Work> ProcessGroupB200::endCoalescing() {
  if (hostsim() || !arena_) {
    auto work = c10::make_intrusive<WorkB200>(rank_, c10d::OpType::COALESCED, std::vector<at::Tensor>{}, device_, nullptr, timeout_);
    work->finish_host();
    return work;
  }
  // every collective of the group ran on the comm queue, in order: a marker behind them covers them all
  DeviceSwitch sw(device_);
  auto work = make_work(c10d::OpType::COALESCED, {});
  work->notifier_.place(comm_q_);
  return work;
}

// ---- gather / scatter / all-to-all, composed ---------------------------------------------------
c10::intrusive_ptr<c10d::Work> ProcessGroupB200::work_on_current_queue(c10d::OpType op, std::vector<at::Tensor> outputs) {
  if (hostsim()) {
    auto work = c10::make_intrusive<WorkB200>(rank_, op, std::move(outputs), device_, nullptr, timeout_);
    work->finish_host();
    return work;
  }
  auto work = make_work(op, outputs);
  work->keep_alive_ = std::move(outputs);
  work->notifier_.place(getCurrentQueue(device_));
  return work;
}

at::Tensor ProcessGroupB200::gather_all(const at::Tensor& mine) {
  at::Tensor flat = mine.contiguous().view({-1});
  at::Tensor all = at::empty({size_, flat.numel()}, flat.options());
  at::Tensor out_flat = all.view({-1});
  _allgather_base(out_flat, flat, c10d::AllgatherOptions())->wait();  // the current queue waits for the exchange
  return all;
}

c10::intrusive_ptr<c10d::Work> ProcessGroupB200::gather(std::vector<std::vector<at::Tensor>>& outputs,
                                                        std::vector<at::Tensor>& inputs, const c10d::GatherOptions& opts) {
  check_single(inputs);
  const int root = static_cast<int>(opts.rootRank);
  TORCH_CHECK(root >= 0 && root < size_, "bwccl gather: invalid root rank ", root);
  if (rank_ == root) {
    TORCH_CHECK(outputs.size() == 1 && static_cast<int>(outputs[0].size()) == size_,
                "bwccl gather: the root passes one list of world-size output tensors");
    for (auto& o : outputs[0])
      TORCH_CHECK(o.numel() == inputs[0].numel() && o.scalar_type() == inputs[0].scalar_type(),
                  "bwccl gather: every output must have the input's size and dtype");
  } else {
    TORCH_CHECK(outputs.empty() || outputs[0].empty(), "bwccl gather: only the root passes output tensors");
  }
  at::Tensor all = gather_all(inputs[0]);
  std::vector<at::Tensor> outs;
  if (rank_ == root) {
    for (int r = 0; r < size_; ++r) {
      outputs[0][r].copy_(all[r].view(outputs[0][r].sizes()));
      outs.push_back(outputs[0][r]);
    }
  }
  return work_on_current_queue(c10d::OpType::GATHER, outs);
}

c10::intrusive_ptr<c10d::Work> ProcessGroupB200::scatter(std::vector<at::Tensor>& outputs,
                                                         std::vector<std::vector<at::Tensor>>& inputs,
                                                         const c10d::ScatterOptions& opts) {
  check_single(outputs);
  const int root = static_cast<int>(opts.rootRank);
  TORCH_CHECK(root >= 0 && root < size_, "bwccl scatter: invalid root rank ", root);
  at::Tensor& out = outputs[0];
  at::Tensor flat = at::empty({size_, out.numel()}, out.options());
  if (rank_ == root) {
    TORCH_CHECK(inputs.size() == 1 && static_cast<int>(inputs[0].size()) == size_,
                "bwccl scatter: the root passes one list of world-size input tensors");
    for (int r = 0; r < size_; ++r) {
      TORCH_CHECK(inputs[0][r].numel() == out.numel() && inputs[0][r].scalar_type() == out.scalar_type(),
                  "bwccl scatter: every input must have the output's size and dtype");
      flat[r].copy_(inputs[0][r].reshape({-1}));
    }
  } else {
    TORCH_CHECK(inputs.empty() || inputs[0].empty(), "bwccl scatter: only the root passes input tensors");
  }
  std::vector<at::Tensor> one{flat};
  c10d::BroadcastOptions bo;
  bo.rootRank = root;
  broadcast(one, bo)->wait();
  out.copy_(flat[rank_].view(out.sizes()));
  return work_on_current_queue(c10d::OpType::SCATTER, {out});
}

c10::intrusive_ptr<c10d::Work> ProcessGroupB200::alltoall_base(at::Tensor& output, at::Tensor& input,
                                                               std::vector<int64_t>& output_splits,
                                                               std::vector<int64_t>& input_splits, const c10d::AllToAllOptions&) {
  TORCH_CHECK(is_b200(output) && is_b200(input), "bwccl all_to_all: tensors must live on the blackwell device");
  ensure_arena(input.device().index());
  TORCH_CHECK(output_splits.empty() && input_splits.empty(), "bwccl all_to_all: only equal splits are implemented");
  TORCH_CHECK(input.numel() % size_ == 0 && output.numel() == input.numel() && output.scalar_type() == input.scalar_type(),
              "bwccl all_to_all: input and output must have the same size, divisible by the world size");
  const int64_t chunk = input.numel() / size_;
  at::Tensor all = gather_all(input);                                   // [world, world * chunk]
  at::Tensor mine = all.view({size_, size_, chunk}).select(1, rank_);   // chunk `rank` of every rank's input
  if (output.is_contiguous()) output.view({size_, chunk}).copy_(mine);
  else output.copy_(mine.reshape(output.sizes()));
  return work_on_current_queue(c10d::OpType::ALLTOALL_BASE, {output});
}

c10::intrusive_ptr<c10d::Work> ProcessGroupB200::alltoall(std::vector<at::Tensor>& outputs, std::vector<at::Tensor>& inputs,
                                                          const c10d::AllToAllOptions&) {
  TORCH_CHECK(static_cast<int>(outputs.size()) == size_ && static_cast<int>(inputs.size()) == size_,
              "bwccl all_to_all: one input and one output tensor per rank expected");
  const int64_t chunk = inputs[0].numel();
  for (int r = 0; r < size_; ++r) {
    TORCH_CHECK(is_b200(inputs[r]) && is_b200(outputs[r]), "bwccl all_to_all: tensors must live on the blackwell device");
    TORCH_CHECK(inputs[r].numel() == chunk && outputs[r].numel() == chunk && inputs[r].scalar_type() == inputs[0].scalar_type() &&
                    outputs[r].scalar_type() == inputs[0].scalar_type(),
                "bwccl all_to_all: only tensors of one size and dtype are implemented");
  }
  ensure_arena(inputs[0].device().index());
  at::Tensor flat = at::empty({size_, chunk}, inputs[0].options());
  for (int r = 0; r < size_; ++r) flat[r].copy_(inputs[r].reshape({-1}));
  at::Tensor all = gather_all(flat).view({size_, size_, chunk});
  for (int r = 0; r < size_; ++r) outputs[r].copy_(all[r][rank_].view(outputs[r].sizes()));
  return work_on_current_queue(c10d::OpType::ALLTOALL, outputs);
}

// ---- fused DDP path -------------------------------------------------------------------------
// The bucket kernel's steps on the host, for ranks that talk through the Store (host simulation): (cast the local
// fp32 gradients to the exchange dtype and clear them) -> sum over ranks in fp32 -> scale -> optimizer update of this
// rank's shard of the parameters, with the same arithmetic as opt_update() in the device code -> every rank receives
// every shard (fp32 and the optional 16-bit copy) -> gradients cleared.  Optimizer state exists for the own shard only.
void ProcessGroupB200::hostsim_fused_step(const at::Tensor& grads, const at::Tensor& params, const at::Tensor& state1,
                                          const at::Tensor& state2, int64_t kind, double lr, double momentum, double dampening,
                                          double weight_decay, double beta1, double beta2, double eps, int64_t step, bool nesterov,
                                          bool first_step, double scale, const std::optional<at::Tensor>& lowp,
                                          const std::optional<at::Tensor>& cast_src, bool zero_grads, int64_t shard) {
  const int64_t n = grads.numel();
  const bool has_src = cast_src.has_value() && cast_src->defined();
  at::Tensor mine;
  if (has_src) {
    TORCH_CHECK(cast_src->scalar_type() == at::kFloat && cast_src->numel() >= n && grads.scalar_type() != at::kFloat,
                "fused_allreduce_step: cast_src must be fp32 and the exchange dtype 16-bit");
    mine = cast_src->narrow(0, 0, n).to(grads.scalar_type());  // rounded once, as in the exchange region
    cast_src->zero_();
  } else {
    mine = grads;
  }
  auto all = store_exchange(to_bytes(mine), true, 0);
  at::Tensor total = at::zeros({n}, at::TensorOptions().dtype(at::kFloat));
  for (auto& b : all) total.add_(from_bytes(b, mine).to(at::kFloat));
  const float* g = total.data_ptr<float>();
  const int64_t begin = std::min<int64_t>(n, (int64_t)rank_ * shard), end = std::min<int64_t>(n, begin + shard);
  // params / state live in host memory under host simulation
  at::Tensor pc = params.cpu().contiguous();
  float* w = pc.data_ptr<float>();
  at::Tensor s1 = state1.cpu().contiguous(), s2 = state2.defined() && state2.numel() ? state2.cpu().contiguous() : at::Tensor();
  float* m1 = s1.data_ptr<float>();
  float* m2 = s2.defined() ? s2.data_ptr<float>() : nullptr;
  const float flr = (float)lr, fmom = (float)momentum, fdamp = (float)dampening, fwd = (float)weight_decay, fb1 = (float)beta1,
              fb2 = (float)beta2, feps = (float)eps, fscale = (float)scale;
  const float bc1 = kind == 1 ? (float)(1.0 - std::pow(beta1, (double)step)) : 1.f;
  const float bc2_sqrt = kind == 1 ? (float)std::sqrt(1.0 - std::pow(beta2, (double)step)) : 1.f;
  for (int64_t i = begin; i < end; ++i) {
    const int64_t s = i - begin;
    float d = g[i] * fscale, wk = w[i];
    if (kind == 0) {
      d += fwd * wk;
      if (fmom != 0.f) {
        const float b = first_step ? d : fmom * m1[s] + (1.f - fdamp) * d;
        m1[s] = b;
        d = nesterov ? d + fmom * b : b;
      }
      w[i] = wk - flr * d;
    } else {
      TORCH_CHECK(m2 != nullptr, "fused_allreduce_step: AdamW needs the second-moment state");
      wk *= 1.f - flr * fwd;
      const float a = fb1 * m1[s] + (1.f - fb1) * d;
      const float v = fb2 * m2[s] + (1.f - fb2) * d * d;
      m1[s] = a;
      m2[s] = v;
      w[i] = wk - (flr / bc1) * (a / (std::sqrt(v) / bc2_sqrt + feps));
    }
  }
  state1.copy_(s1);
  if (s2.defined()) state2.copy_(s2);
  // all-gather of the updated shards (every rank sends `shard` elements; the last one may be partly padding)
  at::Tensor out_shard = at::zeros({shard}, at::TensorOptions().dtype(at::kFloat));
  if (end > begin) out_shard.narrow(0, 0, end - begin).copy_(pc.narrow(0, begin, end - begin));
  auto shards = store_exchange(to_bytes(out_shard), true, 0);
  for (int r = 0; r < size_; ++r) {
    const int64_t b0 = std::min<int64_t>(n, (int64_t)r * shard), e0 = std::min<int64_t>(n, b0 + shard);
    if (e0 > b0) pc.narrow(0, b0, e0 - b0).copy_(from_bytes(shards[r], out_shard).narrow(0, 0, e0 - b0));
  }
  params.copy_(pc);
  if (lowp.has_value() && lowp->defined()) {
    TORCH_CHECK(lowp->numel() == n, "fused_allreduce_step: the 16-bit parameter copy must match the parameters");
    lowp->copy_(pc);
  }
  if (zero_grads && !has_src) grads.zero_();
}

at::Tensor ProcessGroupB200::symm_empty(int64_t numel, at::ScalarType dtype) {
  ensure_arena(device_ >= 0 ? device_ : current_device());
  if (hostsim()) {
    // no peer mapping under host simulation (messages travel through the Store): an ordinary tensor, padded like
    // the real one so that every rank's shard fits
    at::Tensor t = at::empty({numel + 16 * size_}, at::TensorOptions().dtype(dtype).device(make_device(device_)));
    return t.narrow(0, 0, numel);
  }
  TORCH_CHECK(arena_, "symm_empty needs an initialised arena");
  const size_t bytes = static_cast<size_t>(numel) * c10::elementSize(dtype);
  const size_t off = arena_->user_alloc(bytes + 16 * size_);  // room for shard padding
  void* ptr = arena_->local() + off;
  c10::DataPtr dp(ptr, nullptr, [](void*) {}, make_device(device_));
  auto storage = c10::make_intrusive<c10::StorageImpl>(c10::StorageImpl::use_byte_size_t(), bytes, std::move(dp), nullptr, false);
  at::Tensor t = at::detail::make_tensor<B200TensorImpl>(c10::Storage(std::move(storage)),
                                                         c10::DispatchKeySet(c10::DispatchKey::PrivateUse1),
                                                         c10::scalarTypeToTypeMeta(dtype));
  t.unsafeGetTensorImpl()->set_sizes_contiguous({numel});
  return t;
}

int64_t ProcessGroupB200::shard_elems(int64_t numel, at::ScalarType dtype) const {
  return b200_comm_shard_elems(numel, size_, dtype_code(dtype));
}

c10::intrusive_ptr<c10d::Work> ProcessGroupB200::fused_allreduce_step(
    const at::Tensor& grads, const at::Tensor& params, const at::Tensor& state1, const at::Tensor& state2, int64_t kind,
    double lr, double momentum, double dampening, double weight_decay, double beta1, double beta2, double eps,
    int64_t step, bool nesterov, bool first_step, double scale, const std::optional<at::Tensor>& lowp,
    const std::optional<at::Tensor>& cast_src, bool zero_grads) {
  TORCH_CHECK(params.scalar_type() == at::kFloat && grads.numel() == params.numel(), "fused_allreduce_step: params must be fp32 and match grads");
  const int64_t shard = shard_elems(grads.numel(), grads.scalar_type());
  TORCH_CHECK(state1.scalar_type() == at::kFloat && state1.numel() >= shard, "fused_allreduce_step: state shard too small");
  if (hostsim()) {
    ensure_arena(grads.device().index());
    return hostsim_collective(c10d::OpType::ALLREDUCE, {grads, params, state1}, [&] {
      hostsim_fused_step(grads, params, state1, state2, kind, lr, momentum, dampening, weight_decay, beta1, beta2, eps, step, nesterov,
                         first_step, scale, lowp, cast_src, zero_grads, shard);
    });
  }
  TORCH_CHECK(arena_, "fused_allreduce_step needs an initialised arena");
  const size_t goff = arena_->offset_of(grads.data_ptr()), poff = arena_->offset_of(params.data_ptr());
  B200FusedOptArgs o;
  std::memset(&o, 0, sizeof(o));
  o.kind = (int)kind;
  o.lr = (float)lr; o.momentum = (float)momentum; o.dampening = (float)dampening; o.weight_decay = (float)weight_decay;
  o.beta1 = (float)beta1; o.beta2 = (float)beta2; o.eps = (float)eps;
  o.bc1 = kind == 1 ? (float)(1.0 - std::pow(beta1, (double)step)) : 1.f;
  o.bc2_sqrt = kind == 1 ? (float)std::sqrt(1.0 - std::pow(beta2, (double)step)) : 1.f;
  o.nesterov = nesterov; o.first_step = first_step;
  o.state1 = state1.data_ptr<float>();
  o.state2 = state2.defined() && state2.numel() ? state2.data_ptr<float>() : nullptr;
  std::vector<at::Tensor> used{grads, params, state1};
  if (lowp.has_value() && lowp->defined()) {
    TORCH_CHECK(lowp->numel() == params.numel() && (lowp->scalar_type() == at::kBFloat16 || lowp->scalar_type() == at::kHalf),
                "fused_allreduce_step: the 16-bit parameter copy must match the parameters");
    o.lowp_offset = arena_->offset_of(lowp->data_ptr());
    o.lowp_dtype = dtype_code(lowp->scalar_type());
    used.push_back(*lowp);
  }
  if (cast_src.has_value() && cast_src->defined()) {
    TORCH_CHECK(cast_src->scalar_type() == at::kFloat && cast_src->numel() >= shard * size_ && grads.scalar_type() != at::kFloat &&
                    is_b200(*cast_src) && cast_src->is_contiguous(),
                "fused_allreduce_step: cast_src must be a padded fp32 device tensor and the exchange dtype 16-bit");
    o.cast_src = cast_src->data_ptr<float>();
    used.push_back(*cast_src);
  }
  o.zero_grads = zero_grads ? 1 : 0;
  return run_on_comm(c10d::OpType::ALLREDUCE, used, [&, goff, poff, o](void* stream) {
    const B200CommCtx ctx = arena_->ctx();
    COMM_CHECK(b200_comm_allreduce_opt(&ctx, goff, poff, grads.numel(), dtype_code(grads.scalar_type()), (float)scale, &o,
                                       ++seq_, stream));
  });
}

void ProcessGroupB200::set_wait_limit_ms(int64_t ms) {
  // remembered when the arena does not exist yet (it is created by the first collective)
  wait_limit_ms_ = ms;
  apply_wait_limit();
}
void ProcessGroupB200::setTimeout(std::chrono::milliseconds timeout) {
  timeout_ = timeout;
  apply_wait_limit();
}
// Device-side waits run out after the explicit limit if one was set, else after the group's own
// timeout (init_process_group(timeout=...)): a peer that is late by less than that (a checkpoint
// save on rank 0, a slow first step) must not poison the communicator.
void ProcessGroupB200::apply_wait_limit() {
  if (!arena_) return;
  const int64_t ms = wait_limit_ms_ > 0 ? wait_limit_ms_ : static_cast<int64_t>(timeout_.count());
  arena_->set_timeout_ns(ms > 0 ? static_cast<unsigned long long>(ms) * 1000000ull : 0ull);
}
bool ProcessGroupB200::multicast_enabled() {
  ensure_arena(device_ >= 0 ? device_ : current_device());
  return arena_ && arena_->multicast();
}
int64_t ProcessGroupB200::status_word() const { return arena_ ? *((volatile int*)arena_->status_host()) : 0; }
void ProcessGroupB200::clear_status() {
  if (!arena_) return;
  // A kernel in which only some CTAs gave up leaves the CTA-arrival counter of the end barrier
  // non-zero; it has to start from zero again or the next collective signals "done" early.
  DeviceSwitch sw(device_);
  comm_q_.synchronize();
  COMM_CHECK(b200_memset_async(arena_->counter_ptr(), 0, 16, nullptr));  // both CTA counters
  COMM_CHECK(b200_device_synchronize());
  *((volatile int*)arena_->status_host()) = 0;
  status_logged_.store(false);
}

}  // namespace catch_b200
