#include "graph.h"

#include <c10/util/Exception.h>

#include "backend.h"
#include "caching_allocator.h"
#include "device.h"

namespace catch_b200 {

namespace {
thread_local int t_capture_depth = 0;
}

bool graphCaptureActive() { return t_capture_depth > 0; }

DeviceGraph::~DeviceGraph() {
  try {
    if (capturing_) capture_abort();
    reset();
  } catch (...) {
  }
}

void DeviceGraph::capture_begin() {
  TORCH_CHECK(backend().supports_graphs(), "b200 graphs need a device (the host simulation runs work when it is submitted)");
  TORCH_CHECK(!capturing_ && !exec_, "b200 graph: already captured; call reset() first");
  TORCH_CHECK(t_capture_depth == 0, "b200 graph: captures do not nest");
  device_ = current_device();
  queue_ = getCurrentQueue(device_);
  TORCH_CHECK(queue_.handle() != nullptr,
              "b200 graph: the default queue cannot be captured; make a queue from the pool current first");
  pool_ = newPrivatePool();
  backend().graph_begin_capture(queue_.handle());
  prev_pool_ = setThreadPrivatePool(pool_);
  capturing_ = true;
  ++t_capture_depth;
}

bool DeviceGraph::capture_end() {
  TORCH_CHECK(capturing_, "b200 graph: capture_end without capture_begin");
  capturing_ = false;
  --t_capture_depth;
  setThreadPrivatePool(prev_pool_);
  DeviceSwitch sw(device_);
  exec_ = backend().graph_end_capture(queue_.handle(), &num_nodes_);
  if (!exec_) {
    retirePrivatePool(pool_);
    pool_ = 0;
    return false;
  }
  return true;
}

void DeviceGraph::capture_abort() {
  if (!capturing_) return;
  capturing_ = false;
  --t_capture_depth;
  setThreadPrivatePool(prev_pool_);
  DeviceSwitch sw(device_);
  int nodes = 0;
  void* exec = backend().graph_end_capture(queue_.handle(), &nodes);
  if (exec) backend().graph_destroy(exec);
  retirePrivatePool(pool_);
  pool_ = 0;
}

void DeviceGraph::replay() {
  TORCH_CHECK(exec_, "b200 graph: nothing captured");
  DeviceSwitch sw(device_);
  backend().graph_launch(exec_, getCurrentQueue(device_).handle());
}

void DeviceGraph::reset() {
  if (exec_) {
    DeviceSwitch sw(device_);
    // launches still in flight read the pool's memory: let them finish before the pool is shared
    synchronize(device_);
    backend().graph_destroy(exec_);
    exec_ = nullptr;
  }
  if (pool_) {
    retirePrivatePool(pool_);
    pool_ = 0;
  }
  num_nodes_ = 0;
}

}  // namespace catch_b200
