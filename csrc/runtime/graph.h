// Executable device graphs: a sequence of launches captured once from a queue and replayed with one
// submission.  Launch-bound loops (small-batch inference, fusion groups of many short kernels) spend
// more host time submitting kernels than the GPU spends running them; a replay costs one launch.
//
// Memory: everything allocated between capture_begin() and capture_end() comes from a pool private to
// the graph, so addresses baked into the captured launches stay valid (and unshared) until the graph
// is destroyed.  Tensors created during capture and still alive afterwards are the graph's static
// outputs: every replay overwrites them.  Inputs must be tensors that exist before the capture and
// keep their storage; new data is copied into them before a replay.
#pragma once
#include <cstdint>

#include "queue.h"

namespace catch_b200 {

class DeviceGraph {
 public:
  DeviceGraph() = default;
  ~DeviceGraph();
  DeviceGraph(const DeviceGraph&) = delete;
  DeviceGraph& operator=(const DeviceGraph&) = delete;

  // Starts capturing the current queue of the current device, which must not be the default queue.
  void capture_begin();
  // Ends the capture.  Returns false (and leaves the graph empty) when the captured region contained
  // something that cannot be replayed, e.g. a call that waits for the device.
  bool capture_end();
  // Aborts a capture after an exception inside the captured region.
  void capture_abort();
  void replay();  // on the current queue of the graph's device
  void reset();
  bool valid() const { return exec_ != nullptr; }
  int num_nodes() const { return num_nodes_; }

 private:
  void* exec_ = nullptr;
  uint64_t pool_ = 0;
  uint64_t prev_pool_ = 0;
  int device_ = -1;
  int num_nodes_ = 0;
  bool capturing_ = false;
  Queue queue_;
};

// True while the calling thread is between capture_begin() and capture_end(): code that would wait for
// the device or time kernels with events skips that part.
bool graphCaptureActive();

}  // namespace catch_b200
