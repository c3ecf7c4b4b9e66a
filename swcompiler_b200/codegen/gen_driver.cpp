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
//   A name with the suffix _fused (mlp8_fused, convnet_fused, resblock_fused) selects tensor-core precision and the
//   emit-time fusion planner: one call per fused chain, bf16 activations between fused calls.
//
// Needs a reference checkout to compile (swcompiler_b200/codegen/build_codegen.py).
#include <fstream>
#include <iostream>
#include <string>
#include <vector>

#include "B200Codegen.h"
#include "SWC.h"

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

}  // namespace

int main(int argc, char **argv) {
    if (argc < 4) {
        std::cerr << "usage: gen_driver mlp8|convnet|resblock[_fused] <out_dir> <repo_root>\n";
        return 2;
    }
    const std::string which = argv[1], out_dir = argv[2], repo = argv[3];
    const std::string suffix = "_fused";
    const bool fused = which.size() > suffix.size() && which.compare(which.size() - suffix.size(), suffix.size(), suffix) == 0;
    const std::string base = fused ? which.substr(0, which.size() - suffix.size()) : which;
    IRGraph *g = base == "mlp8" ? build_mlp8() : (base == "convnet" ? build_convnet() : (base == "resblock" ? build_resblock() : nullptr));
    if (!g) {
        std::cerr << "unknown graph " << base << "\n";
        return 2;
    }
    Config config;  // inference, one device, no MPI: the defaults
    g->setConfig(config);
    Engine engine(g);
    engine.compile();  // the reference's own passes: labeling, FC lowering, renaming
    swcb200::B200Codegen gen(g, config, /*device=*/0, /*precision=*/fused ? 1 : 0, /*fuse=*/fused);
    engine.setCodegenerator(&gen);
    const std::string code = engine.genCode();
    std::ofstream(out_dir + "/" + which + "_Graph.cpp") << code;
    std::ofstream(out_dir + "/" + which + "_Makefile") << gen.makefileText(repo);
    std::cerr << which << ": " << gen.arenaBytes() << " bytes of device arena, " << gen.fusedGroups() << " fused calls\n";
    return 0;
}
