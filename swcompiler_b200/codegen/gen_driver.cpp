// gen_driver: builds an inference graph with the reference's public API, runs the reference's Engine
// passes on it unchanged, installs B200Codegen as the generator and writes the emitted program.
//
//   gen_driver mlp8    <out_dir> <repo_root>   the 8-image MNIST MLP of the reference's fixture set
//                                              (784-512-10, tanh, softmax, top-3)
//   gen_driver convnet <out_dir> <repo_root>   Conv3x3 -> BatchNorm -> Add(skip) -> ReLU -> MaxPool -> FC ->
//                                              Softmax -> top-1 on [4,8,8,4] inputs read from files
//   gen_driver resblock <out_dir> <repo_root>  [2,8,8,64] -> Conv3x3 -> BN -> ReLU -> Conv3x3 -> BN -> Add(skip) -> ReLU ->
//                                              MaxPool -> FC -> Softmax -> top-1: a residual block wide enough (64
//                                              channels) for the tensor-core convolution
//   gen_driver mlp_eval <out_dir> <repo_root>  the MLP inside a streaming evaluation loop: batches of 4 from a record file
//                                              (config.use_dataloader), top-1, running accuracy counters
//   gen_driver fcpair   <out_dir> <repo_root>  [64,256] -> FC 256->512 -> ReLU -> FC 512->128, no bias: the model-parallel
//                                              pair (only meaningful with _mp<N>)
//   gen_driver resproj  <out_dir> <repo_root>  a residual block with a projection shortcut on [2,8,8,64]: main branch
//                                              Conv3x3 -> BN -> ReLU -> Conv3x3 -> BN, shortcut Conv1x1 -> BN, then
//                                              Add -> ReLU -> MaxPool -> FC -> Softmax -> top-1 (two branches meet at the add)
//   gen_driver convact  <out_dir> <repo_root>  [2,8,8,64] -> Conv2dWithActivation(3x3, ReLU) -> MaxPool -> FC -> Softmax -> top-1
//   gen_driver badop    <out_dir> <repo_root>  a graph with an op outside the kernel table (ElementMul): the generator
//                                              must refuse it (exit code 3, #error in the text)
//   gen_driver c2lenet  <out_dir> <repo_root>  a Caffe2 model read by Caffe2Import from c2lenet_predict.pb / c2lenet_init.pb in
//   gen_driver c2resnet <out_dir> <repo_root>  the working directory (tests/golden/caffe2_models.py writes them); the weight
//                                              files the import produces go to the working directory too
//   A name with _dp<N> (mlp8_dp2) partitions the graph over N ranks by the batch: config.mpi, config.mpi_size = N,
//   config.force_data_parallel, the reference's ParallelLabeling / ParallelLowering passes unchanged.
//   A name with _mp<N> (fcpair_mp2, mlp8_mp2) sets the model-parallel strategies by hand -- first FC split by output
//   columns {-1,1,1}, the activation on column tiles {1,1}, second FC by input rows {1,0,-2}; for the MLP the bias-adds
//   on row tiles, which makes the passes insert Transform nodes -- and runs ParallelLowering on them (the labeling pass
//   draws strategies from std::random_device, so it is skipped for a reproducible program).
//   A name with _rp<N> leaves the choice to the reference's labeling pass, which draws from std::random_device: every run
//   gives another partitioning (used to fuzz the generator, not for committed samples).
//   A name that ends in _graph (mlp8_graph, convnet_fused_graph) has the forward pass captured into a CUDA graph and
//   replayed three times.
//   A name with the suffix _fused (mlp8_fused, convnet_fused, resblock_fused) selects tensor-core precision and the
//   emit-time fusion planner: one call per fused chain, bf16 activations between fused calls.
//
// Needs a reference checkout to compile (swcompiler_b200/codegen/build_codegen.py).
#include <fstream>
#include <iostream>
#include <string>
#include <vector>

#include "B200Codegen.h"
#include "Caffe2Import.h"
#include "SWC.h"
#include "pass/EliminationPass.h"
#include "pass/ParallelLoweringPass.h"
#include "pass/RenamingNodePass.h"

using namespace swc;
using namespace swc::op;

namespace {

TensorNode *tensor(IRGraph *g, const std::string &name, std::initializer_list<size_t> dims, const char *file = nullptr,
                   DataType dt = DataType::Float_t) {
    auto *t = new Tensor(dims, dt);
    if (file) t->setTensorInit(TensorInitType::FILE, file);
    auto *n = new TensorNode(name, t);
    g->pushTensorNode(n);
    return n;
}

template <typename... Parents> OpNode *op(IRGraph *g, const std::string &name, Op *o, Parents... parents) {
    auto *n = new OpNode(name, o);
    n->exlinkUpperNode(parents...);
    g->pushOpNode(n);
    return n;
}

TensorNode *result(IRGraph *g, const std::string &name, std::initializer_list<size_t> dims, OpNode *producer,
                   DataType dt = DataType::Float_t) {
    auto *n = tensor(g, name, dims, nullptr, dt);
    n->exlinkUpperNode(producer);
    return n;
}

IRGraph *build_mlp8() {
    auto *g = new IRGraph();
    auto *x = tensor(g, "data0", {8, 784}, "mnist_images_8.bin");
    auto *w0 = tensor(g, "weight0", {784, 512}, "mlp_weight0.bin");
    auto *b0 = tensor(g, "bias0", {512}, "mlp_bias0.bin");
    auto *fc0 = op(g, "fc0", new MatrixMatrixFCBiasOp(), x, w0, b0);
    auto *h0 = result(g, "data1", {8, 512}, fc0);
    auto *th = op(g, "tanh0", new MatrixTanhOp(), h0);
    auto *h1 = result(g, "data2", {8, 512}, th);
    auto *w1 = tensor(g, "weight1", {512, 10}, "mlp_weight1.bin");
    auto *b1 = tensor(g, "bias1", {10}, "mlp_bias1.bin");
    auto *fc1 = op(g, "fc1", new MatrixMatrixFCBiasOp(), h1, w1, b1);
    auto *logits = result(g, "data3", {8, 10}, fc1);
    auto *sm = op(g, "softmax", new MatrixSoftmaxOp(), logits);
    auto *probs = result(g, "data4", {8, 10}, sm);
    auto *am = op(g, "argmax", new ArgMaxOp(3), probs);
    auto *top3 = result(g, "top3", {8, 3}, am, DataType::Int32_t);
    g->findInOut();
    g->updateTopology();
    g->addDisplayTensorNodes(probs, top3);
    return g;
}

IRGraph *build_convnet() {
    auto *g = new IRGraph();
    std::vector<size_t> k3{3, 3}, s1{1, 1}, p1{1, 1, 1, 1}, k2{2, 2}, s2{2, 2}, p0{0, 0, 0, 0};
    auto *x = tensor(g, "image", {4, 8, 8, 4}, "cn_input.bin");
    auto *cw = tensor(g, "conv_w", {4, 3, 3, 4}, "cn_conv_w.bin");
    auto *cb = tensor(g, "conv_b", {4}, "cn_conv_b.bin");
    auto *conv = op(g, "conv0", new Conv2dOp(k3, s1, p1), x, cw, cb);
    auto *c0 = result(g, "conv_out", {4, 8, 8, 4}, conv);
    auto *sc = tensor(g, "bn_scale", {4}, "cn_bn_scale.bin");
    auto *bi = tensor(g, "bn_bias", {4}, "cn_bn_bias.bin");
    auto *me = tensor(g, "bn_mean", {4}, "cn_bn_mean.bin");
    auto *va = tensor(g, "bn_var", {4}, "cn_bn_var.bin");
    auto *bn = op(g, "bn0", new BatchNormalizationOp(1e-5f), c0, sc, bi, me, va);
    auto *n0 = result(g, "bn_out", {4, 8, 8, 4}, bn);
    auto *add = op(g, "add0", new ElementAddOp(), n0, x);
    auto *a0 = result(g, "add_out", {4, 8, 8, 4}, add);
    auto *relu = op(g, "relu0", new ReluOp(), a0);
    auto *r0 = result(g, "relu_out", {4, 8, 8, 4}, relu);
    auto *pool = op(g, "pool0", new MaxPoolOp(k2, s2, p0), r0);
    auto *q0 = result(g, "pool_out", {4, 4, 4, 4}, pool);
    auto *fw = tensor(g, "fc_w", {64, 10}, "cn_fc_w.bin");
    auto *fb = tensor(g, "fc_b", {10}, "cn_fc_b.bin");
    auto *fc = op(g, "fc0", new MatrixMatrixFCBiasOp(), q0, fw, fb);
    auto *logits = result(g, "logits", {4, 10}, fc);
    auto *sm = op(g, "softmax", new MatrixSoftmaxOp(), logits);
    auto *probs = result(g, "probs", {4, 10}, sm);
    auto *am = op(g, "argmax", new ArgMaxOp(1), probs);
    auto *top1 = result(g, "top1", {4, 1}, am, DataType::Int32_t);
    g->findInOut();
    g->updateTopology();
    g->addDisplayTensorNodes(probs, top1);
    return g;
}

// The MNIST MLP as a streaming evaluation: batches of 4 from a record file, top-1, running accuracy
// (the graph of the reference's test/engine/testEngineMLPInfer.cpp).
IRGraph *build_mlp_eval() {
    auto *g = new IRGraph();
    auto *x = tensor(g, "data0", {4, 784});
    auto *w0 = tensor(g, "weight0", {784, 512}, "mlp_weight0.bin");
    auto *b0 = tensor(g, "bias0", {512}, "mlp_bias0.bin");
    auto *fc0 = op(g, "fc0", new MatrixMatrixFCBiasOp(), x, w0, b0);
    auto *h0 = result(g, "data1", {4, 512}, fc0);
    auto *th = op(g, "tanh0", new MatrixTanhOp(), h0);
    auto *h1 = result(g, "data2", {4, 512}, th);
    auto *w1 = tensor(g, "weight1", {512, 10}, "mlp_weight1.bin");
    auto *b1 = tensor(g, "bias1", {10}, "mlp_bias1.bin");
    auto *fc1 = op(g, "fc1", new MatrixMatrixFCBiasOp(), h1, w1, b1);
    auto *logits = result(g, "data3", {4, 10}, fc1);
    auto *sm = op(g, "softmax", new MatrixSoftmaxOp(), logits);
    auto *probs = result(g, "data4", {4, 10}, sm);
    auto *am = op(g, "argmax", new ArgMaxOp(1), probs);
    auto *top1 = result(g, "top1", {4, 1}, am, DataType::Int32_t);
    auto *label = tensor(g, "selected", {4}, nullptr, DataType::Int32_t);
    auto *acc = op(g, "accuracy", new AccuracyOp(), top1, label);
    auto *accur = result(g, "accur", {1, 2}, acc, DataType::Int32_t);
    accur->getTensor()->setTensorInit(TensorInitType::CONSTANT, 0);
    g->findInOut();
    g->updateTopology();
    g->setInferDataNodes(label, x);
    g->addDisplayTensorNodes(accur);
    return g;
}

IRGraph *build_fcpair() {
    auto *g = new IRGraph();
    auto *x = tensor(g, "x", {64, 256}, "fp_x.bin");
    auto *w1 = tensor(g, "w1", {256, 512}, "fp_w1.bin");
    auto *fc1 = op(g, "fc1", new MatrixMatrixFCOp(), x, w1);
    auto *h = result(g, "h", {64, 512}, fc1);
    auto *relu = op(g, "relu", new ReluOp(), h);
    auto *hr = result(g, "hr", {64, 512}, relu);
    auto *w2 = tensor(g, "w2", {512, 128}, "fp_w2.bin");
    auto *fc2 = op(g, "fc2", new MatrixMatrixFCOp(), hr, w2);
    auto *y = result(g, "y", {64, 128}, fc2);
    g->findInOut();
    g->updateTopology();
    g->addDisplayTensorNodes(y);
    return g;
}

IRGraph *build_resblock() {
    auto *g = new IRGraph();
    std::vector<size_t> k3{3, 3}, s1{1, 1}, p1{1, 1, 1, 1}, k2{2, 2}, s2{2, 2}, p0{0, 0, 0, 0};
    auto *x = tensor(g, "image", {2, 8, 8, 64}, "rb_input.bin");
    TensorNode *cur = x;
    TensorNode *bn_out[2];
    for (int i = 0; i < 2; i++) {
        const std::string n = std::to_string(i);
        auto *cw = tensor(g, "conv" + n + "_w", {64, 3, 3, 64}, ("rb_conv" + n + "_w.bin").c_str());
        auto *cb = tensor(g, "conv" + n + "_b", {64}, ("rb_conv" + n + "_b.bin").c_str());
        auto *conv = op(g, "conv" + n, new Conv2dOp(k3, s1, p1), cur, cw, cb);
        auto *c = result(g, "conv" + n + "_out", {2, 8, 8, 64}, conv);
        auto *sc = tensor(g, "bn" + n + "_scale", {64}, ("rb_bn" + n + "_scale.bin").c_str());
        auto *bi = tensor(g, "bn" + n + "_bias", {64}, ("rb_bn" + n + "_bias.bin").c_str());
        auto *me = tensor(g, "bn" + n + "_mean", {64}, ("rb_bn" + n + "_mean.bin").c_str());
        auto *va = tensor(g, "bn" + n + "_var", {64}, ("rb_bn" + n + "_var.bin").c_str());
        auto *bn = op(g, "bn" + n, new BatchNormalizationOp(1e-5f), c, sc, bi, me, va);
        bn_out[i] = result(g, "bn" + n + "_out", {2, 8, 8, 64}, bn);
        if (i == 0) {
            auto *relu = op(g, "relu0", new ReluOp(), bn_out[0]);
            cur = result(g, "relu0_out", {2, 8, 8, 64}, relu);
        }
    }
    auto *add = op(g, "add1", new ElementAddOp(), bn_out[1], x);
    auto *a1 = result(g, "add1_out", {2, 8, 8, 64}, add);
    auto *relu1 = op(g, "relu1", new ReluOp(), a1);
    auto *r1 = result(g, "relu1_out", {2, 8, 8, 64}, relu1);
    auto *pool = op(g, "pool0", new MaxPoolOp(k2, s2, p0), r1);
    auto *q0 = result(g, "pool_out", {2, 4, 4, 64}, pool);
    auto *fw = tensor(g, "fc_w", {1024, 10}, "rb_fc_w.bin");
    auto *fb = tensor(g, "fc_b", {10}, "rb_fc_b.bin");
    auto *fc = op(g, "fc0", new MatrixMatrixFCBiasOp(), q0, fw, fb);
    auto *logits = result(g, "logits", {2, 10}, fc);
    auto *sm = op(g, "softmax", new MatrixSoftmaxOp(), logits);
    auto *probs = result(g, "probs", {2, 10}, sm);
    auto *am = op(g, "argmax", new ArgMaxOp(1), probs);
    auto *top1 = result(g, "top1", {2, 1}, am, DataType::Int32_t);
    g->findInOut();
    g->updateTopology();
    g->addDisplayTensorNodes(probs, top1);
    return g;
}

// conv -> batch-norm on `in`, returns the batch-norm output; files <prefix><tag>_*.bin
TensorNode *conv_bn(IRGraph *g, TensorNode *in, const std::string &tag, const std::string &prefix, size_t k, size_t pad) {
    std::vector<size_t> kk{k, k}, s1{1, 1}, pp{pad, pad, pad, pad};
    auto *cw = tensor(g, "conv" + tag + "_w", {64, k, k, 64}, (prefix + "conv" + tag + "_w.bin").c_str());
    auto *cb = tensor(g, "conv" + tag + "_b", {64}, (prefix + "conv" + tag + "_b.bin").c_str());
    auto *conv = op(g, "conv" + tag, new Conv2dOp(kk, s1, pp), in, cw, cb);
    auto *c = result(g, "conv" + tag + "_out", {2, 8, 8, 64}, conv);
    auto *sc = tensor(g, "bn" + tag + "_scale", {64}, (prefix + "bn" + tag + "_scale.bin").c_str());
    auto *bi = tensor(g, "bn" + tag + "_bias", {64}, (prefix + "bn" + tag + "_bias.bin").c_str());
    auto *me = tensor(g, "bn" + tag + "_mean", {64}, (prefix + "bn" + tag + "_mean.bin").c_str());
    auto *va = tensor(g, "bn" + tag + "_var", {64}, (prefix + "bn" + tag + "_var.bin").c_str());
    auto *bn = op(g, "bn" + tag, new BatchNormalizationOp(1e-5f), c, sc, bi, me, va);
    return result(g, "bn" + tag + "_out", {2, 8, 8, 64}, bn);
}

// pool 2x2/2 -> FC 1024->10 -> softmax -> top-1 behind a [2,8,8,64] activation; files <prefix>fc_*.bin
void classifier_tail(IRGraph *g, TensorNode *act, const std::string &prefix) {
    std::vector<size_t> k2{2, 2}, s2{2, 2}, p0{0, 0, 0, 0};
    auto *pool = op(g, "pool0", new MaxPoolOp(k2, s2, p0), act);
    auto *q0 = result(g, "pool_out", {2, 4, 4, 64}, pool);
    auto *fw = tensor(g, "fc_w", {1024, 10}, (prefix + "fc_w.bin").c_str());
    auto *fb = tensor(g, "fc_b", {10}, (prefix + "fc_b.bin").c_str());
    auto *fc = op(g, "fc0", new MatrixMatrixFCBiasOp(), q0, fw, fb);
    auto *logits = result(g, "logits", {2, 10}, fc);
    auto *sm = op(g, "softmax", new MatrixSoftmaxOp(), logits);
    auto *probs = result(g, "probs", {2, 10}, sm);
    auto *am = op(g, "argmax", new ArgMaxOp(1), probs);
    auto *top1 = result(g, "top1", {2, 1}, am, DataType::Int32_t);
    g->findInOut();
    g->updateTopology();
    g->addDisplayTensorNodes(probs, top1);
}

// A residual block whose shortcut is itself a convolution (1x1 + batch-norm): two convolution chains end at the add.
IRGraph *build_resproj() {
    auto *g = new IRGraph();
    auto *x = tensor(g, "image", {2, 8, 8, 64}, "rp_input.bin");
    auto *shortcut = conv_bn(g, x, "S", "rp_", 1, 0);   // declared first: it also comes first in the topological order
    auto *b0 = conv_bn(g, x, "0", "rp_", 3, 1);
    auto *relu0 = op(g, "relu0", new ReluOp(), b0);
    auto *r0 = result(g, "relu0_out", {2, 8, 8, 64}, relu0);
    auto *b1 = conv_bn(g, r0, "1", "rp_", 3, 1);
    auto *add = op(g, "add1", new ElementAddOp(), b1, shortcut);
    auto *a1 = result(g, "add1_out", {2, 8, 8, 64}, add);
    auto *relu1 = op(g, "relu1", new ReluOp(), a1);
    auto *r1 = result(g, "relu1_out", {2, 8, 8, 64}, relu1);
    classifier_tail(g, r1, "rp_");
    return g;
}

IRGraph *build_convact() {
    auto *g = new IRGraph();
    std::vector<size_t> k3{3, 3}, s1{1, 1}, p1{1, 1, 1, 1};
    auto *x = tensor(g, "image", {2, 8, 8, 64}, "ca_input.bin");
    auto *cw = tensor(g, "conv_w", {64, 3, 3, 64}, "ca_conv_w.bin");
    auto *cb = tensor(g, "conv_b", {64}, "ca_conv_b.bin");
    auto *conv = op(g, "conv0", new Conv2dWithActivationOp(k3, s1, p1, SWC_ACTIVATION_RELU), x, cw, cb);
    auto *c = result(g, "conv_out", {2, 8, 8, 64}, conv);
    classifier_tail(g, c, "ca_");
    return g;
}

// A Caffe2 model: predict and init net from the working directory, top-1 behind the model's softmax.
IRGraph *build_caffe2(const std::string &model) {
    auto *g = new IRGraph();
    auto *data = model == "c2lenet" ? new TensorNode("data", {4, 28, 28, 1}) : new TensorNode("data", {2, 8, 8, 64});
    data->getTensor()->setTensorInit(TensorInitType::FILE, model + "_input.bin");
    swcb200::Caffe2Import imp(g, model + "_predict.pb", model + "_init.pb", {data}, ".", model + "_");
    if (!imp.ok()) {
        std::cerr << "import of " << model << " failed: " << imp.error() << "\n";
        exit(4);
    }
    TensorNode *probs = imp.output();
    const size_t rows = probs->getDims()[0];
    auto *am = op(g, "argmax", new ArgMaxOp(1), probs);
    auto *top1 = result(g, "top1", {rows, 1}, am, DataType::Int32_t);
    g->findInOut();
    g->updateTopology();
    g->addDisplayTensorNodes(probs, top1);
    return g;
}

// an op the kernel table has no entry for, in the middle of a forward pass
IRGraph *build_badop() {
    auto *g = new IRGraph();
    auto *x = tensor(g, "x", {4, 16}, "bo_x.bin");
    auto *y = tensor(g, "y", {4, 16}, "bo_y.bin");
    auto *mul = op(g, "mul0", new ElementMulOp(), x, y);
    auto *m = result(g, "prod", {4, 16}, mul);
    auto *sm = op(g, "softmax", new MatrixSoftmaxOp(), m);
    auto *probs = result(g, "probs", {4, 16}, sm);
    g->findInOut();
    g->updateTopology();
    g->addDisplayTensorNodes(probs);
    return g;
}

}  // namespace

int main(int argc, char **argv) {
    if (argc < 4) {
        std::cerr << "usage: gen_driver mlp8|convnet|resblock|fcpair[_dp<N>|_mp<N>][_fused] <out_dir> <repo_root>\n";
        return 2;
    }
    const std::string which = argv[1], out_dir = argv[2], repo = argv[3];
    // name = <graph>[_dp<N> | _mp<N>][_fused][_graph]
    std::string base = which;
    auto strip = [&base](const std::string &suffix) {
        if (base.size() <= suffix.size() || base.compare(base.size() - suffix.size(), suffix.size(), suffix) != 0) return false;
        base = base.substr(0, base.size() - suffix.size());
        return true;
    };
    const bool graph = strip("_graph");
    const bool fused = strip("_fused");
    int ranks = 1;
    bool model_parallel = false;
    bool random_strategies = false;  // _rp<N>: whatever the reference's labeling pass draws (not reproducible: for fuzzing)
    for (const char *tag : {"_dp", "_mp", "_rp"}) {
        const size_t at = base.rfind(tag);
        if (at != std::string::npos && at + 3 < base.size() && isdigit(base[at + 3])) {
            ranks = atoi(base.c_str() + at + 3);
            model_parallel = std::string(tag) == "_mp";
            random_strategies = std::string(tag) == "_rp";
            base = base.substr(0, at);
        }
    }
    IRGraph *g = base == "mlp8" ? build_mlp8()
                 : base == "convnet" ? build_convnet()
                 : base == "resblock" ? build_resblock()
                 : base == "fcpair" ? build_fcpair()
                 : base == "mlp_eval" ? build_mlp_eval()
                 : base == "resproj" ? build_resproj()
                 : base == "convact" ? build_convact()
                 : (base == "c2lenet" || base == "c2resnet") ? build_caffe2(base)
                 : base == "badop" ? build_badop() : nullptr;
    if (!g) {
        std::cerr << "unknown graph " << base << "\n";
        return 2;
    }
    Config config;  // inference, one device, no MPI: the defaults
    if (base == "mlp_eval") {
        config.use_dataloader = true;
        config.dataloader_src = "mnist8_records.bin";
        config.label_bytes = BytesProto::ONE_BYTE_AS_INT;
        config.data_bytes = BytesProto::FOUR_BYTES_AS_FLOAT;
        config.dataloader_samples = 10;  // 8 images + 2 more: batches of 4 use 8, the tail is dropped
    }
    if (ranks > 1) {
        config.mpi = true;
        config.mpi_size = ranks;
        config.force_data_parallel = !model_parallel && !random_strategies;
    }
    g->setConfig(config);
    Engine engine(g);
    if (!model_parallel) {
        engine.compile();  // the reference's own passes: labeling, FC lowering, renaming (+ the parallel passes)
    } else {
        engine.runInferPasses();
        g->resetParallelStrategy();
        auto label = [&](const char *name, std::vector<int> strategy) {
            auto *n = dynamic_cast<OpNode *>(g->getNodeByName(name));
            if (!n) {
                std::cerr << "no op node " << name << "\n";
                exit(2);
            }
            n->setStrategyLabel(new StrategyLabel(strategy));
        };
        if (base == "fcpair") {
            label("fc1_mm", {-1, 1, 1});
            label("relu", {1, 1});
            label("fc2_mm", {1, 0, -2});
        } else if (base == "mlp8") {
            // column-split first FC, bias-add on row tiles (a 1 -> 0 re-tiling), tanh on column tiles (0 -> 1),
            // row-split second FC (partial sums, Reduce), the rest on row tiles
            label("fc0_mm", {-1, 1, 1});
            label("fc0_add", {0, -1, 0});
            label("tanh0", {1, 1});
            label("fc1_mm", {1, 0, -2});
            label("fc1_add", {0, -1, 0});
            label("softmax", {0, 0});
            label("argmax", {0, 0});
        } else {
            std::cerr << "no model-parallel strategies written down for " << base << "\n";
            return 2;
        }
        pass::ParallelLoweringPass(g).run();
        pass::RenamingNodePass(g).run();
        pass::EliminationPass(g).run();
        g->findInOut();
        g->updateTopology();
    }
    swcb200::B200Codegen gen(g, config, /*device=*/0, /*precision=*/fused ? 1 : 0, /*fuse=*/fused, /*graph_replays=*/graph ? 3 : 0);
    engine.setCodegenerator(&gen);
    const std::string code = engine.genCode();
    std::ofstream(out_dir + "/" + which + "_Graph.cpp") << code;
    std::ofstream(out_dir + "/" + which + "_Makefile") << gen.makefileText(repo);
    std::cerr << which << ": " << gen.arenaBytes() << " bytes of device arena, " << gen.fusedGroups() << " fused calls\n";
    if (!gen.unsupportedOps().empty()) {
        for (const std::string &u : gen.unsupportedOps()) std::cerr << "cannot emit: " << u << "\n";
        return 3;  // the text written above holds an #error for each: it does not compile
    }
    return 0;
}
