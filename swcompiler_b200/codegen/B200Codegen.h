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
// With `fuse` (and tensor-core precision) the generator plans at emit time: it matches the chains the
// lowering pass leaves behind -- MatrixMatrixMul -> MatrixVectorAdd -> Tanh/Relu, and
// Conv2d -> BatchNormalization -> ElementAdd -> Relu -- and prints ONE fused table call for each
// (swcb200_fc_bf16, swcb200_conv2d_bf16).  Weights and filters are packed to bf16 once after loading,
// activations that only fused calls read are kept in bf16, and casts are printed only where an fp32
// consumer (an unfused op, a displayed tensor) meets a bf16 producer or the other way round.
//
// Partitioned graphs (config.mpi with config.mpi_size ranks, after the reference's ParallelLabeling and
// ParallelLowering passes): the program is printed once and run as one process per GPU.  Where the
// reference's ParallelCodegen prints MPI text for the Scatter / Gather / Reduce / Transform nodes
// (src/codegen/ParallelCodegen.cpp:457-896) this generator prints swcb200_scatter / _gather /
// _reduce_sum / _transform (NCCL over NVLink).  Tensors the passes label "master" (device rank 0) live in
// an arena only rank 0 allocates; tiles and replicas live in every rank's arena; an op whose tensors are
// not on every rank is printed inside `if (rank == 0)`, as the reference does (:959-1006).  The ranks
// find each other without MPI: rank and count come from the environment, the NCCL id through a file.
//
// With config.use_dataloader (IRGraph::setInferDataNodes, config.dataloader_src / _samples / data_bytes) the forward
// pass is printed inside a streaming evaluation loop over a record file, the counterpart of the reference's
// `while (loader.next(label, data))` (src/codegen/Codegen.cpp:930-995): double-buffered pinned host buffers and
// device slots, uploads on a second stream, AccuracyOp -> swcb200_accuracy_i.
//
// This header needs the reference's headers on the include path (-I<reference>/src); it is compiled
// only where a reference checkout is present (swcompiler_b200/codegen/build_codegen.py).
#pragma once

#include <map>
#include <string>
#include <vector>

#include "common.h"
#include "codegen/Codegen.h"

namespace swc {
class IRNode;
}

namespace swcb200 {

class B200Codegen : public swc::codegen::Codegen {
  public:
    // precision: 0 = strict fp32 (bit-exact with the reference's generated C), 1 = tensor-core bf16 for the
    // fp32 entry points (see swc_b200.h)
    // fuse: plan fused calls as described above (ignored in strict precision: there are no fused strict kernels)
    // graph_replays > 0: the forward pass is captured into a CUDA graph after one plain run and launched that many
    // times (for forward passes that are bound by launch latency; single-GPU programs without a data loader)
    B200Codegen(swc::IRGraph *graph, Config &config, int device = 0, int precision = 0, bool fuse = false,
                int graph_replays = 0);

    void emitHeader() override;
    void emitEnvInit() override;
    void emitEnvFinalize() override;
    void allocateMemAddr() override;
    void emitVarDeclarations() override;
    void emitMemAllocations() override;
    void emitTensorAddresses() override;
    void emitTensorInitializations() override;
    void emitInferDataLoaderInit() override {}  // the loader is set up where the evaluation loop is printed (emitExecute)
    void emitExecute() override;
    void emitFuncCalls() override;
    void emitMemFree() override;

    // text of the Makefile that builds the emitted program against the kernel library
    std::string makefileText(const std::string &repo_root) const;
    size_t arenaBytes() const { return arena_bytes_; }

    // number of fused calls planned (after genCode)
    int fusedGroups() const { return (int)groups_.size(); }
    // ops the kernel table cannot carry out (after genCode).  Not empty: the emitted text holds an #error for each
    // and must not be used.
    const std::vector<std::string> &unsupportedOps() const { return unsupported_; }

  private:
    // A chain of op nodes printed as one call.  Intermediate tensors of the chain are never materialised.
    struct Group {
        enum Kind { FC, CONV } kind;
        std::vector<swc::OpNode *> ops;      // in chain order; ops[0] is the head
        swc::Tensor *in = nullptr;           // A (FC) / input image (conv)
        swc::Tensor *weight = nullptr;       // W[k,n] (FC) / filter [oC,kh,kw,iC] (conv)
        swc::Tensor *bias = nullptr;         // may be null for FC
        swc::Tensor *bn[4] = {nullptr, nullptr, nullptr, nullptr};  // scale, bias, mean, var
        float bn_eps = 0.f;
        swc::Tensor *skip = nullptr;         // residual
        int act = 0;                         // 0 none, 1 relu, 2 tanh
        swc::Tensor *out = nullptr;          // the chain's last tensor
        // A row-split FC whose partial products a Reduce node sums: the pair is printed as the peer-memory join
        // (the GEMM's epilogue stores each row block into its owner's slots, the owners add, the master gathers).
        // Conv chain followed by MaxPool 2x2 / 2 where the row-interleaved convolution kernel runs: the pool is the
        // last step of the fused call's epilogue.
        swc::OpNode *pool = nullptr;         // the MaxPool node
        swc::Tensor *conv_out = nullptr;     // the convolution's own (un-pooled) result: its dims go into the call
        swc::OpNode *join = nullptr;         // the Reduce node
        swc::Tensor *join_out = nullptr;     // its result, on the master
    };
    void planFusion();
    bool matchFc(swc::OpNode *op, Group &g);
    bool matchConv(swc::OpNode *op, Group &g);
    bool needsF32(swc::Tensor *t);
    bool availableBefore(swc::IRNode *tensor_node, swc::OpNode *head);
    void unsupported(swc::OpNode *op, const std::string &why, std::ostream &os);
    void walk(bool dry);                     // prints (or, dry, only records) the calls of the forward pass
    void emitGroup(const Group &g, std::ostream &os, bool dry);
    void ensureF32(swc::Tensor *t, std::ostream &os);
    void ensureBf16(swc::Tensor *t, std::ostream &os);
    swc::Tensor *root(swc::Tensor *t);       // the tensor a view (Reshape) finally aliases
    std::string bf16Name(swc::Tensor *t) { return nameOf(root(t)) + "_bf16"; }
    std::string packedName(swc::Tensor *t) { return nameOf(t) + "_packed"; }
    std::string dimsArrayTo(std::ostream &os, const std::string &name, const std::vector<size_t> &dims);

    void emitOp(swc::OpNode *op);
    void emitOpTo(swc::OpNode *op, std::ostream &os);
    void emitPrintOutputs();
    std::string dimsArray(const std::string &name, const std::vector<size_t> &dims);
    std::string nameOf(swc::Tensor *t) { return tensors_name_map_[t]; }
    // the fp32 storage a tensor is read from: its own, or, for a view in a fused plan, the viewed tensor's
    std::string f32Name(swc::Tensor *t) { return fuse_ ? nameOf(root(t)) : nameOf(t); }

    // partitioned graphs
    bool onEveryRank(swc::IRNode *tensor_node);
    bool runsOnEveryRank(swc::OpNode *op);
    bool isLoadTimeScatter(swc::OpNode *op);
    bool isConstant(swc::IRNode *tensor_node);
    bool isLoaderFed(swc::Tensor *t);
    void emitCommOp(swc::OpNode *op, std::ostream &os);
    void emitGuarded(swc::OpNode *op, std::ostream &os);   // the op's call, inside `if (rank == 0)` where it must be

    int device_, precision_;
    bool fuse_;
    int graph_replays_ = 0;
    bool parallel_ = false;
    int nranks_ = 1;
    size_t master_bytes_ = 0;
    std::map<swc::Tensor *, bool> on_master_;
    std::vector<std::string> unsupported_;
    std::vector<Group> groups_;
    std::map<swc::OpNode *, int> group_of_;          // op node -> index into groups_
    std::map<swc::Tensor *, swc::Tensor *> alias_;     // view -> viewed
    std::map<swc::Tensor *, bool> have_f32_, have_bf16_;   // state of the walk, keyed by root tensor
    std::map<swc::Tensor *, bool> made_f32_, made_bf16_;   // what the dry walk materialised (drives the arena plan)
    std::map<swc::Tensor *, size_t> bf16_offsets_, packed_offsets_;
    std::vector<swc::Tensor *> bf16_order_, packed_order_;
    int join_group_ = -1;                              // the one group printed as a peer-memory join, if any
    size_t join_rows_offset_ = 0, join_meet_offset_ = 0;
    std::string joinSlots() { return nameOf(root(groups_[join_group_].out)); }   // the p slots: the partial-sum tensor's storage
    size_t arena_bytes_ = 0, stage_bytes_ = 0;
    std::map<swc::Tensor *, size_t> offsets_;
    std::vector<swc::Tensor *> order_;  // tensors in the order they were placed
    int array_counter_ = 0;
};

}  // namespace swcb200
