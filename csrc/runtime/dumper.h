// Op-level tensor dump tool.
//
// Parity: DumpTool of the reference (torch_mlu/csrc/aten/util/cndumper.h:41-268,
// Python side torch_mlu/core/dumptool.py:34-91): while dumping is active every
// operator that touches a device tensor gets a directory "<k>_<op>" (nested for ops
// called inside ops) holding one text file per tensor argument ("dev_<i>") and
// result ("dev_result_<i>"; with use_cpu also "cpu_result_<i>", the same op re-run on
// CPU copies of the arguments).  File format: a header line
//   Tensor : Type = Float : Shape = [2, 3] : Stride = [3, 1] : Dumped = 6
// followed by one value per line.  Level 0 dumps the first 10 values, level 1 the sum
// of absolute values, level 2 everything.
#pragma once
#include <string>

namespace catch_b200 {

void dump_start(const std::string& dir, bool enable, bool use_cpu, int level);
void dump_finish();
bool dump_running();

}  // namespace catch_b200
