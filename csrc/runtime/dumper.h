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

// Kernel case generator.  Parity: the reference hands this to its kernel library
// (torch_mlu/core/dumptool.py:34-73 -> cnnlSetGenCaseMode): every library call writes a
// reproducible description of itself.  Here every dispatcher operator that touches a
// device tensor writes one JSON case file "<dir>/<op>/<op>_<n>.json" with its schema, the
// dtype / shape / stride / memory format of each tensor argument and the value of every
// other argument.  Level 1: descriptions only; 2: also the tensor bytes ("<case>.arg<i>.bin",
// slow); 3: descriptions printed to stderr, no files; 0: off.  catch_b200.dumptool.replay_case
// re-runs a case on the device and on the CPU.
void gencase_set(int level, const std::string& dir);
int gencase_level();

}  // namespace catch_b200
