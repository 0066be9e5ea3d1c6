// TorchScript fusion mode of the b200 backend.
//
// Parity with the reference's JIT layer (torch_mlu/csrc/jit/**): a global toggle
// (interface.cpp:36-45); a lowering pre-pass (inline, drop exception-only branches,
// remove dropout / contiguous, constant-fold, CSE, DCE -- lower/passes/magicmind/*.cpp);
// a partitioner that greedily merges supported nodes into fusion-group subgraph nodes
// with alias-safe moves (partition/passes/segment_graph.cpp:102-244); a registered
// fusion-group operator whose runner is cached by (graph, argument dtypes / shapes /
// device) and falls back to the plain interpreter on failure
// (runtime/graph_runner.cpp:108-238, runner_cache.cpp:44-85).
// Instead of a vendor graph compiler, "compiling" a group means rewriting its
// conv(+folded BN)+ReLU(+residual) and linear(+bias)+activation chains into this
// backend's fused tcgen05 ops (catch_b200::conv_bn_act / linear_act).
#pragma once
#include <torch/csrc/jit/ir/ir.h>
#include <memory>
#include <string>

namespace catch_b200 {
namespace jit {

bool fusion_enabled();
void set_fusion_enabled(bool on);

// Passes (usable directly on a graph, e.g. from tests).
void LowerGraph(std::shared_ptr<torch::jit::Graph>& graph);
void FuseKernels(std::shared_ptr<torch::jit::Graph>& graph);   // pattern rewrite to fused ops
void SegmentGraph(std::shared_ptr<torch::jit::Graph>& graph);  // build FusionGroup nodes
void UnfuseGraph(std::shared_ptr<torch::jit::Graph>& graph);   // dissolve them again (needed before saving a module)
bool isSupported(const torch::jit::Node* n);

void register_passes();  // idempotent: registers the pre-passes with the graph executor
int64_t fusion_cache_size();
void fusion_cache_clear();
int64_t fusion_compile_count();
int64_t fusion_fallback_count();
int64_t fusion_graph_capture_count();  // fusion groups captured as device graphs
int64_t fusion_graph_replay_count();

}  // namespace jit
}  // namespace catch_b200
