// B200Codegen -- a code generator for SWCompiler graphs that targets the swc_b200 kernel table.
//
// It plugs into the reference unchanged: derive from swc::codegen::Codegen, install with
// Engine::setCodegenerator (src/engine/Engine.h:39) and call Engine::genCode().  The graph IR, the op
// classes and the passes are used as they are; only what is PRINTED changes.  Where the reference's
// generator prints `#include "utils/kernels.h"` and one scalar-loop call per op node
// (src/codegen/Codegen.cpp:221-286, :1035-1132, :1171-2494), this one prints `#include "swc_b200.h"`
// and one `swcb200_*` call per op node, places every tensor in ONE device arena with 256-byte aligned
// offsets, stages file-initialised tensors through a host buffer, and synchronises before results are
// read back and printed.
//
// This header needs the reference's headers on the include path (-I<reference>/src); it is compiled
// only where a reference checkout is present (swcompiler_b200/codegen/build_codegen.py).
#pragma once

#include <map>
#include <string>
#include <vector>

#include "common.h"
#include "codegen/Codegen.h"

namespace swcb200 {

class B200Codegen : public swc::codegen::Codegen {
  public:
    // precision: 0 = strict fp32 (bit-exact with the reference's generated C), 1 = tensor-core bf16 for the
    // fp32 entry points (see swc_b200.h)
    B200Codegen(swc::IRGraph *graph, Config &config, int device = 0, int precision = 0);

    void emitHeader() override;
    void emitEnvInit() override;
    void emitEnvFinalize() override;
    void allocateMemAddr() override;
    void emitVarDeclarations() override;
    void emitMemAllocations() override;
    void emitTensorAddresses() override;
    void emitTensorInitializations() override;
    void emitExecute() override;
    void emitFuncCalls() override;
    void emitMemFree() override;

    // text of the Makefile that builds the emitted program against the kernel library
    std::string makefileText(const std::string &repo_root) const;
    size_t arenaBytes() const { return arena_bytes_; }

  private:
    void emitOp(swc::OpNode *op);
    void emitPrintOutputs();
    std::string dimsArray(const std::string &name, const std::vector<size_t> &dims);
    std::string nameOf(swc::Tensor *t) { return tensors_name_map_[t]; }

    int device_, precision_;
    size_t arena_bytes_ = 0, stage_bytes_ = 0;
    std::map<swc::Tensor *, size_t> offsets_;
    std::vector<swc::Tensor *> order_;  // tensors in the order they were placed
    int array_counter_ = 0;
};

}  // namespace swcb200
