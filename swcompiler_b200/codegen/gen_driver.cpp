// gen_driver: builds an inference graph with the reference's public API, runs the reference's Engine
// passes on it unchanged, installs B200Codegen as the generator and writes the emitted program.
//
//   gen_driver mlp8    <out_dir> <repo_root>   the 8-image MNIST MLP of the reference's fixture set
//                                              (784-512-10, tanh, softmax, top-3)
//   gen_driver convnet <out_dir> <repo_root>   Conv3x3 -> BatchNorm -> Add(skip) -> ReLU -> MaxPool -> FC ->
//                                              Softmax -> top-1 on [4,8,8,4] inputs read from files
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

}  // namespace

int main(int argc, char **argv) {
    if (argc < 4) {
        std::cerr << "usage: gen_driver mlp8|convnet <out_dir> <repo_root>\n";
        return 2;
    }
    const std::string which = argv[1], out_dir = argv[2], repo = argv[3];
    IRGraph *g = which == "mlp8" ? build_mlp8() : build_convnet();
    Config config;  // inference, one device, no MPI: the defaults
    g->setConfig(config);
    Engine engine(g);
    engine.compile();  // the reference's own passes: labeling, FC lowering, renaming
    swcb200::B200Codegen gen(g, config, /*device=*/0, /*precision=*/0);
    engine.setCodegenerator(&gen);
    const std::string code = engine.genCode();
    std::ofstream(out_dir + "/" + which + "_Graph.cpp") << code;
    std::ofstream(out_dir + "/" + which + "_Makefile") << gen.makefileText(repo);
    std::cerr << which << ": " << gen.arenaBytes() << " bytes of device arena\n";
    return 0;
}
