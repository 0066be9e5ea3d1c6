// torch.distributed backend of the b200 device ("bwccl").
//
// Capability parity with ProcessGroupCNCL (torch_mlu/csrc/distributed/
// process_group_cncl.{hpp,cpp}): one process per device; collectives run on a
// dedicated communication queue that is ordered against the compute queue with
// notifiers (no host blocking); tensors handed to a collective are recorded on the
// comm queue so the caching allocator does not recycle them early; bootstrap goes
// through the c10d Store.  Differences on purpose: the transport is this project's
// own kernels over peer-mapped memory (comm.cu) instead of a vendor library;
// timeouts are honoured and device-side wait failures surface as exceptions (the
// reference ignores the timeout and never reports asynchronous errors,
// process_group_cncl.cpp:107-115,583-589); reduce_scatter / _allgather_base /
// allreduce_coalesced are implemented.
// Under host simulation the same class moves bytes through the Store, so rank
// logic, ordering, time-outs and failure handling are testable without GPUs.
#pragma once
#include <atomic>
#include <condition_variable>
#include <deque>
#include <mutex>
#include <thread>
#include <torch/csrc/distributed/c10d/Backend.hpp>
#include <torch/csrc/distributed/c10d/Store.hpp>
#include <torch/csrc/distributed/c10d/Work.hpp>

#include <atomic>
#include <memory>

#include "../device/kernels_api.h"
#include "../runtime/notifier.h"
#include "../runtime/queue.h"

namespace catch_b200 {

class SymmetricArena;

class WorkB200 : public c10d::Work {
 public:
  WorkB200(int rank, c10d::OpType op, std::vector<at::Tensor> outputs, int device, int* status,
           std::chrono::milliseconds timeout);
  bool isCompleted() override;
  bool isSuccess() const override;
  std::exception_ptr exception() const override;
  bool wait(std::chrono::milliseconds timeout = kNoTimeout) override;
  void synchronize() override;
  std::vector<at::Tensor> result() override { return outputs_; }
  c10::intrusive_ptr<c10::ivalue::Future> getFuture() override;
  void finish_host(std::exception_ptr err = nullptr);  // host-only work (hostsim / errors)

  Notifier notifier_{/*enable_timing=*/false};
  std::vector<at::Tensor> keep_alive_;

 private:
  void check_status() const;
  std::vector<at::Tensor> outputs_;
  int device_;
  int* status_;
  std::chrono::milliseconds timeout_;
  bool host_done_ = false;
  std::exception_ptr error_;
  c10::intrusive_ptr<c10::ivalue::Future> future_;
};

class ProcessGroupB200 : public c10d::Backend {
 public:
  ProcessGroupB200(const c10::intrusive_ptr<c10d::Store>& store, int rank, int size, std::chrono::milliseconds timeout);
  ~ProcessGroupB200() override;

  const std::string getBackendName() const override { return "bwccl"; }
  void setTimeout(std::chrono::milliseconds timeout) override;

  c10::intrusive_ptr<c10d::Work> broadcast(std::vector<at::Tensor>& tensors, const c10d::BroadcastOptions& opts) override;
  c10::intrusive_ptr<c10d::Work> allreduce(std::vector<at::Tensor>& tensors, const c10d::AllreduceOptions& opts) override;
  c10::intrusive_ptr<c10d::Work> allreduce_coalesced(std::vector<at::Tensor>& tensors,
                                                     const c10d::AllreduceCoalescedOptions& opts) override;
  c10::intrusive_ptr<c10d::Work> reduce(std::vector<at::Tensor>& tensors, const c10d::ReduceOptions& opts) override;
  c10::intrusive_ptr<c10d::Work> allgather(std::vector<std::vector<at::Tensor>>& outputs, std::vector<at::Tensor>& inputs,
                                           const c10d::AllgatherOptions& opts) override;
  c10::intrusive_ptr<c10d::Work> _allgather_base(at::Tensor& output, at::Tensor& input,
                                                 const c10d::AllgatherOptions& opts) override;
  c10::intrusive_ptr<c10d::Work> reduce_scatter(std::vector<at::Tensor>& outputs,
                                                std::vector<std::vector<at::Tensor>>& inputs,
                                                const c10d::ReduceScatterOptions& opts) override;
  c10::intrusive_ptr<c10d::Work> _reduce_scatter_base(at::Tensor& output, at::Tensor& input,
                                                      const c10d::ReduceScatterOptions& opts) override;
  // gather / scatter / all-to-all are composed from all-gather and broadcast (every rank receives everything and
  // keeps its part): correct and built from the collectives above, not bandwidth-optimal.  Equal sizes only.
  c10::intrusive_ptr<c10d::Work> gather(std::vector<std::vector<at::Tensor>>& outputs, std::vector<at::Tensor>& inputs,
                                        const c10d::GatherOptions& opts) override;
  c10::intrusive_ptr<c10d::Work> scatter(std::vector<at::Tensor>& outputs, std::vector<std::vector<at::Tensor>>& inputs,
                                         const c10d::ScatterOptions& opts) override;
  c10::intrusive_ptr<c10d::Work> alltoall_base(at::Tensor& output, at::Tensor& input, std::vector<int64_t>& output_splits,
                                               std::vector<int64_t>& input_splits, const c10d::AllToAllOptions& opts) override;
  c10::intrusive_ptr<c10d::Work> alltoall(std::vector<at::Tensor>& outputs, std::vector<at::Tensor>& inputs,
                                          const c10d::AllToAllOptions& opts) override;
  // Coalescing (torch.distributed._coalescing_manager): collectives between the two calls are launched as they come
  // (the comm queue keeps their order); endCoalescing returns one Work that completes after all of them.
  void startCoalescing() override {}
  c10::intrusive_ptr<c10d::Work> endCoalescing() override;
  c10::intrusive_ptr<c10d::Work> send(std::vector<at::Tensor>& tensors, int dst, int tag) override;
  c10::intrusive_ptr<c10d::Work> recv(std::vector<at::Tensor>& tensors, int src, int tag) override;
  c10::intrusive_ptr<c10d::Work> barrier(const c10d::BarrierOptions& opts) override;

  // ---- fused DDP path -------------------------------------------------------------
  // A tensor that lives in this rank's arena at the same offset on every rank.
  at::Tensor symm_empty(int64_t numel, at::ScalarType dtype);
  // reduce-scatter of `grads` (a symm_empty tensor) * scale, optimizer step on this
  // rank's shard of `params` (a symm_empty fp32 tensor), all-gather of the parameters.
  // lowp: symm_empty 16-bit copy of the parameters, refreshed on every rank in the same pass.
  // cast_src: local fp32 gradients (padded to shard_elems * world) that the kernel first converts into
  // `grads` (16-bit), so that only 16-bit values cross NVLink.  zero_grads: the kernel leaves the
  // gradients (cast_src if given, else `grads`) cleared for the next backward pass.
  c10::intrusive_ptr<c10d::Work> fused_allreduce_step(const at::Tensor& grads, const at::Tensor& params,
                                                      const at::Tensor& state1, const at::Tensor& state2, int64_t kind,
                                                      double lr, double momentum, double dampening, double weight_decay,
                                                      double beta1, double beta2, double eps, int64_t step,
                                                      bool nesterov, bool first_step, double scale,
                                                      const std::optional<at::Tensor>& lowp = std::nullopt,
                                                      const std::optional<at::Tensor>& cast_src = std::nullopt,
                                                      bool zero_grads = false);
  int64_t shard_elems(int64_t numel, at::ScalarType dtype) const;
  // all-reduce in place on a symm_empty tensor (no staging copies)
  c10::intrusive_ptr<c10d::Work> allreduce_symm(const at::Tensor& t, int64_t op, double scale, bool test_no_signal);
  void set_wait_limit_ms(int64_t ms);
  int64_t status_word() const;
  void clear_status();
  int device_index() const { return device_; }
  // True when the arena is bound to an NVSwitch multicast object (in-switch reductions are in use).
  bool multicast_enabled();
  // Rank whose heartbeat stopped (it left without saying goodbye), or -1.  Set by the watchdog thread.
  int64_t dead_peer() const { return dead_peer_.load(); }

 private:
  void ensure_arena(int device);
  void apply_wait_limit();
  void check_single(const std::vector<at::Tensor>& tensors) const;
  c10::intrusive_ptr<WorkB200> make_work(c10d::OpType op, std::vector<at::Tensor> outputs);
  // a Work for results that were produced on the current compute queue (composed collectives)
  c10::intrusive_ptr<c10d::Work> work_on_current_queue(c10d::OpType op, std::vector<at::Tensor> outputs);
  // [world, numel] tensor holding every rank's `mine` (flattened), ordered on the current compute queue
  at::Tensor gather_all(const at::Tensor& mine);
  // runs fn(stream) on the comm queue ordered after the current compute queue
  template <typename F>
  c10::intrusive_ptr<c10d::Work> run_on_comm(c10d::OpType op, std::vector<at::Tensor> tensors, F&& fn, Queue* q = nullptr);
  void throw_if_failed() const;
  void gather_into(const at::Tensor& in, const std::vector<char*>& dsts, void* stream);
  // host-simulated transport
  std::vector<std::vector<uint8_t>> store_exchange(const std::vector<uint8_t>& mine, bool everyone_sends, int root);
  c10::intrusive_ptr<c10d::Work> hostsim_collective(c10d::OpType op, std::vector<at::Tensor> outs,
                                                    std::function<void()> fn);
  void hostsim_fused_step(const at::Tensor& grads, const at::Tensor& params, const at::Tensor& state1, const at::Tensor& state2,
                          int64_t kind, double lr, double momentum, double dampening, double weight_decay, double beta1, double beta2,
                          double eps, int64_t step, bool nesterov, bool first_step, double scale,
                          const std::optional<at::Tensor>& lowp, const std::optional<at::Tensor>& cast_src, bool zero_grads,
                          int64_t shard);

  c10::intrusive_ptr<c10d::Store> store_;
  std::chrono::milliseconds timeout_;
  int device_ = -1;
  std::unique_ptr<SymmetricArena> arena_;
  Queue comm_q_, send_q_, recv_q_;
  uint64_t seq_ = 0;
  std::vector<uint64_t> send_seq_, recv_seq_;
  uint64_t host_seq_ = 0;
  std::deque<std::pair<uint64_t, int>> posted_;  // host-simulated transport: (round, extra parts) of messages still in the Store
  int64_t wait_limit_ms_ = 0;     // explicit device-side wait limit (0 = follow timeout_)
  std::string uid_;

  // ---- watchdog: one host thread per group.  It publishes this rank's heartbeat counter in the Store,
  // watches the peers' counters and the device status word, and records a failure so that the next
  // collective raises before anything is launched.
  void start_watchdog();
  void watchdog_loop();
 public:
  // Stops and joins the watchdog thread and posts this rank's goodbye (idempotent).
  void stop_watchdog();
 private:
  std::thread watchdog_;
  std::mutex wd_mu_;
  std::condition_variable wd_cv_;
  bool wd_stop_ = false;
  std::atomic<int64_t> dead_peer_{-1};
  std::atomic<bool> status_logged_{false};
  int64_t hb_interval_ms_ = 1000, hb_timeout_ms_ = 15000;
};

// Stops the watchdog thread of every live group: run at interpreter exit, before static objects (the
// Store server among them) go away under a thread that still uses them.
void stop_all_watchdogs();

// Number of ProcessGroupB200 objects created so far in this process (names Store keys).
int next_process_group_id();

}  // namespace catch_b200
