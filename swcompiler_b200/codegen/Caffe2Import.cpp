// See Caffe2Import.h.
#include "Caffe2Import.h"

#include <algorithm>
#include <cstring>
#include <fstream>
#include <sstream>

#include "SWC.h"

using namespace swc;
using namespace swc::op;

namespace swcb200 {

// ---------------------------------------------------------------------------------------------------
// protobuf wire format: a message is a sequence of (key, value); key = field << 3 | wire type;
// wire types: 0 varint, 1 fixed 64, 2 length-delimited, 5 fixed 32
namespace {

struct Reader {
    const uint8_t *p, *end;
    bool bad;
    Reader(const uint8_t *begin, const uint8_t *stop, bool broken) : p(begin), end(stop), bad(broken) {}
    bool more() const { return !bad && p < end; }
    uint64_t varint() {
        uint64_t v = 0;
        for (int shift = 0; shift < 64; shift += 7) {
            if (p >= end) {
                bad = true;
                return 0;
            }
            const uint8_t b = *p++;
            v |= (uint64_t)(b & 0x7f) << shift;
            if (!(b & 0x80)) return v;
        }
        bad = true;
        return 0;
    }
    Reader sub() {  // a length-delimited field as a reader of its own
        const uint64_t n = varint();
        if (bad || n > (uint64_t)(end - p)) {
            bad = true;
            return Reader{p, p, true};
        }
        Reader r{p, p + n, false};
        p += n;
        return r;
    }
    std::string bytes() {
        Reader r = sub();
        return r.bad ? std::string() : std::string((const char *)r.p, (size_t)(r.end - r.p));
    }
    float fixed32() {
        if (end - p < 4) {
            bad = true;
            return 0.f;
        }
        float f;
        memcpy(&f, p, 4);
        p += 4;
        return f;
    }
    void skip(int wire) {
        switch (wire) {
        case 0: varint(); break;
        case 1: if (end - p < 8) bad = true; else p += 8; break;
        case 2: sub(); break;
        case 5: if (end - p < 4) bad = true; else p += 4; break;
        default: bad = true;
        }
    }
};

void parseArgument(Reader r, PbArgument *a, bool *bad) {
    while (r.more()) {
        const uint64_t key = r.varint();
        const int field = (int)(key >> 3), wire = (int)(key & 7);
        if (field == 1 && wire == 2) {
            a->name = r.bytes();
        } else if (field == 2 && wire == 5) {
            a->f = r.fixed32();
            a->has_f = true;
        } else if (field == 3 && wire == 0) {
            a->i = (int64_t)r.varint();
            a->has_i = true;
        } else if (field == 4 && wire == 2) {
            a->s = r.bytes();
            a->has_s = true;
        } else if (field == 5 && wire == 5) {
            a->floats.push_back(r.fixed32());
        } else if (field == 5 && wire == 2) {  // packed
            Reader q = r.sub();
            while (q.more()) a->floats.push_back(q.fixed32());
            if (q.bad) r.bad = true;
        } else if (field == 6 && wire == 0) {
            a->ints.push_back((int64_t)r.varint());
        } else if (field == 6 && wire == 2) {  // packed
            Reader q = r.sub();
            while (q.more()) a->ints.push_back((int64_t)q.varint());
            if (q.bad) r.bad = true;
        } else {
            r.skip(wire);
        }
    }
    if (r.bad) *bad = true;
}

void parseOperator(Reader r, PbOperator *o, bool *bad) {
    while (r.more()) {
        const uint64_t key = r.varint();
        const int field = (int)(key >> 3), wire = (int)(key & 7);
        if (field == 1 && wire == 2) {
            o->input.push_back(r.bytes());
        } else if (field == 2 && wire == 2) {
            o->output.push_back(r.bytes());
        } else if (field == 3 && wire == 2) {
            o->name = r.bytes();
        } else if (field == 4 && wire == 2) {
            o->type = r.bytes();
        } else if (field == 5 && wire == 2) {
            o->arg.emplace_back();
            parseArgument(r.sub(), &o->arg.back(), bad);
        } else {
            r.skip(wire);
        }
    }
    if (r.bad) *bad = true;
}

}  // namespace

const PbArgument *PbOperator::find(const std::string &n) const {
    for (const PbArgument &a : arg)
        if (a.name == n) return &a;
    return nullptr;
}

bool parseNetDef(const std::string &bytes, PbNet *net, std::string *error) {
    Reader r{(const uint8_t *)bytes.data(), (const uint8_t *)bytes.data() + bytes.size(), false};
    bool bad = false;
    while (r.more()) {
        const uint64_t key = r.varint();
        const int field = (int)(key >> 3), wire = (int)(key & 7);
        if (field == 1 && wire == 2) {
            net->name = r.bytes();
        } else if (field == 2 && wire == 2) {
            net->op.emplace_back();
            parseOperator(r.sub(), &net->op.back(), &bad);
        } else if (field == 7 && wire == 2) {
            net->external_input.push_back(r.bytes());
        } else if (field == 8 && wire == 2) {
            net->external_output.push_back(r.bytes());
        } else {
            r.skip(wire);
        }
    }
    if (r.bad || bad) {
        if (error) *error = "not a serialized NetDef (truncated or malformed field)";
        return false;
    }
    return true;
}

// ---------------------------------------------------------------------------------------------------
namespace {

bool readFile(const std::string &path, std::string *out) {
    std::ifstream f(path, std::ios::in | std::ios::binary);
    if (!f) return false;
    std::ostringstream ss;
    ss << f.rdbuf();
    *out = ss.str();
    return true;
}

// blob names become C identifiers and file names
std::string cleanName(const std::string &blob) {
    std::string n;
    for (char c : blob) n.push_back((isalnum((unsigned char)c) || c == '_') ? c : '_');
    if (n.empty() || isdigit((unsigned char)n[0])) n = "t_" + n;
    return n;
}

// "kernel" / "stride" / "pad" | "pad_t..pad_r" | "pads", as the reference reads them (Caffe2Importer.cpp:36-82)
std::vector<size_t> pair(const PbOperator &op, const char *name, size_t dflt) {
    const PbArgument *a = op.find(name);
    const size_t v = a && a->has_i ? (size_t)a->i : dflt;
    return {v, v};
}
std::vector<size_t> pads(const PbOperator &op) {
    if (const PbArgument *a = op.find("pad")) return std::vector<size_t>(4, (size_t)a->i);
    if (op.find("pad_t")) {
        auto v = [&](const char *n) { const PbArgument *a = op.find(n); return a ? (size_t)a->i : (size_t)0; };
        return {v("pad_t"), v("pad_l"), v("pad_b"), v("pad_r")};
    }
    if (const PbArgument *a = op.find("pads")) {
        std::vector<size_t> p;
        for (int64_t i : a->ints) p.push_back((size_t)i);
        p.resize(4, 0);
        return p;
    }
    return {0, 0, 0, 0};
}
std::vector<size_t> outHW(size_t ih, size_t iw, const std::vector<size_t> &k, const std::vector<size_t> &s, const std::vector<size_t> &p) {
    return {(ih + p[0] + p[2] - k[0]) / s[0] + 1, (iw + p[1] + p[3] - k[1]) / s[1] + 1};
}

Tensor *newTensor(const std::vector<size_t> &dims) {
    auto *shape = new std::vector<unsigned long>(dims.begin(), dims.end());
    return new Tensor(new TensorShape(shape));
}

}  // namespace

bool Caffe2Import::fail(const std::string &why) {
    if (error_.empty()) error_ = why;
    return false;
}

TensorNode *Caffe2Import::tensor(const std::string &blob) const {
    auto it = nodes_.find(blob);
    return it == nodes_.end() ? nullptr : it->second;
}

Caffe2Import::Caffe2Import(IRGraph *graph, const std::string &predict_net_file, const std::string &init_net_file,
                           const std::vector<TensorNode *> &inputs, const std::string &weight_dir,
                           const std::string &weight_prefix)
    : graph_(graph), weight_dir_(weight_dir), weight_prefix_(weight_prefix) {
    for (TensorNode *t : inputs) {
        graph_->pushTensorNode(t);
        nodes_[t->name()] = t;
    }
    std::string bytes, err;
    PbNet init, predict;
    if (!readFile(init_net_file, &bytes)) {
        fail("cannot read " + init_net_file);
        return;
    }
    if (!parseNetDef(bytes, &init, &err)) {
        fail(init_net_file + ": " + err);
        return;
    }
    if (!readFile(predict_net_file, &bytes)) {
        fail("cannot read " + predict_net_file);
        return;
    }
    if (!parseNetDef(bytes, &predict, &err)) {
        fail(predict_net_file + ": " + err);
        return;
    }
    loadWeights(init);
    for (const PbOperator &op : predict.op) {
        if (!ok()) return;
        loadOperator(op);
    }
}

// init_net: one GivenTensorFill / ConstantFill per weight blob (Caffe2Importer.cpp:478-557).  The values are kept in
// memory until the operator that consumes the blob says in which layout it wants them.
void Caffe2Import::loadWeights(const PbNet &init) {
    for (const PbOperator &op : init.op) {
        if (op.output.empty()) continue;
        Blob b;
        if (const PbArgument *shape = op.find("shape"))
            for (int64_t d : shape->ints) b.shape.push_back((size_t)d);
        if (op.type == "GivenTensorFill") {
            if (const PbArgument *v = op.find("values")) b.values = v->floats;
            size_t n = 1;
            for (size_t d : b.shape) n *= d;
            if (b.values.size() != n) {
                fail("GivenTensorFill " + op.output[0] + ": " + std::to_string(b.values.size()) + " values for a shape of " +
                     std::to_string(n));
                return;
            }
        } else if (op.type == "ConstantFill") {
            const PbArgument *v = op.find("value");
            b.constant = true;
            b.fill = v && v->has_f ? v->f : 0.f;
        } else {
            continue;  // UniformFill and the like: not a pretrained weight (the reference skips them too)
        }
        for (const std::string &out : op.output)
            if (!nodes_.count(out)) blobs_[out] = b;
    }
}

// a weight tensor node whose values are written to <weight_dir>/<prefix><name>.bin, in the order given
TensorNode *Caffe2Import::weightNode(const std::string &blob, const std::vector<size_t> &shape, const std::vector<float> &values) {
    const std::string name = cleanName(blob), file = weight_prefix_ + name + ".bin";
    Tensor *t = newTensor(shape);
    std::ofstream f(weight_dir_ + "/" + file, std::ios::out | std::ios::binary);
    f.write((const char *)values.data(), (std::streamsize)(values.size() * sizeof(float)));
    if (!f) {
        fail("cannot write " + weight_dir_ + "/" + file);
        return nullptr;
    }
    t->setTensorInit(TensorInitType::FILE, file);
    auto *node = new TensorNode(name, t);
    graph_->pushTensorNode(node);
    nodes_[blob] = node;
    return node;
}

// a weight used in the layout it came in (biases, batch-norm vectors)
TensorNode *Caffe2Import::plainWeight(const std::string &blob) {
    if (TensorNode *n = tensor(blob)) return n;
    auto it = blobs_.find(blob);
    if (it == blobs_.end()) {
        fail("blob " + blob + " is neither an input nor in the init net");
        return nullptr;
    }
    const Blob &b = it->second;
    if (!b.constant) return weightNode(blob, b.shape, b.values);
    Tensor *t = newTensor(b.shape);
    t->setTensorInit(TensorInitType::CONSTANT, b.fill);
    auto *node = new TensorNode(cleanName(blob), t);
    graph_->pushTensorNode(node);
    nodes_[blob] = node;
    return node;
}

TensorNode *Caffe2Import::result(const std::string &blob, const std::vector<size_t> &dims, OpNode *producer) {
    // Caffe2 nets write in place (Relu: X -> X); every result is a new tensor node here, the blob name moves on to it
    std::string name = cleanName(blob);
    const int seen = op_names_[name + "#t"]++;
    if (nodes_.count(blob) || seen) name += "_v" + std::to_string(seen + 1);
    auto *node = new TensorNode(name, newTensor(dims), producer);
    graph_->pushTensorNode(node);
    nodes_[blob] = node;
    last_output_ = node;
    return node;
}

void Caffe2Import::loadOperator(const PbOperator &op) {
    static const char *supported[] = {"Conv", "SpatialBN", "Relu", "Sum", "MaxPool", "AveragePool", "FC", "Softmax", "Dropout"};
    if (std::find_if(std::begin(supported), std::end(supported), [&](const char *s) { return op.type == s; }) == std::end(supported)) {
        fail("unsupported Caffe2 operator " + op.type);  // the reference exits here (Caffe2Importer.cpp:569-577)
        return;
    }
    if (op.input.empty() || op.output.empty()) {
        fail(op.type + " without input or output");
        return;
    }
    std::string base = op.type;
    std::transform(base.begin(), base.end(), base.begin(), ::tolower);
    const int nth = op_names_[base]++;
    const std::string name = nth ? base + "_" + std::to_string(nth) : base;
    TensorNode *in = tensor(op.input[0]);
    if (!in) {
        fail(op.type + ": input blob " + op.input[0] + " is not defined");
        return;
    }
    const std::vector<size_t> idims = in->getDims();
    OpNode *node = nullptr;

    if (op.type == "Conv") {
        auto wit = blobs_.find(op.input.size() > 1 ? op.input[1] : "");
        if (wit == blobs_.end() || wit->second.shape.size() != 4 || idims.size() != 4) {
            fail("Conv: needs a 4-D input and a 4-D filter from the init net");
            return;
        }
        const Blob &w = wit->second;
        const size_t O = w.shape[0], I = w.shape[1], H = w.shape[2], W = w.shape[3];
        if (I != idims[3]) {
            fail("Conv: filter has " + std::to_string(I) + " input channels, the activation " + std::to_string(idims[3]));
            return;
        }
        // oihw -> ohwi, once
        std::vector<float> v(w.values.size());
        for (size_t o = 0; o < O; o++)
            for (size_t i = 0; i < I; i++)
                for (size_t h = 0; h < H; h++)
                    for (size_t x = 0; x < W; x++) v[((o * H + h) * W + x) * I + i] = w.values[((o * I + i) * H + h) * W + x];
        TensorNode *filter = weightNode(op.input[1], {O, H, W, I}, v);
        TensorNode *bias = nullptr;
        if (op.input.size() >= 3) {
            bias = plainWeight(op.input[2]);
        } else {  // no bias blob: zeros
            Tensor *t = newTensor({O});
            t->setTensorInit(TensorInitType::CONSTANT, 0.f);
            bias = new TensorNode(name + "_bias", t);
            graph_->pushTensorNode(bias);
        }
        if (!filter || !bias) return;
        std::vector<size_t> k = pair(op, "kernel", H), s = pair(op, "stride", 1), p = pads(op);
        node = new OpNode(name, new Conv2dOp(k, s, p));
        node->exlinkUpperNode(in, filter, bias);
        const std::vector<size_t> hw = outHW(idims[1], idims[2], k, s, p);
        result(op.output[0], {idims[0], hw[0], hw[1], O}, node);
    } else if (op.type == "SpatialBN") {
        if (op.input.size() != 5) {
            fail("SpatialBN needs 5 inputs");
            return;
        }
        TensorNode *scale = plainWeight(op.input[1]), *bias = plainWeight(op.input[2]), *mean = plainWeight(op.input[3]),
                   *var = plainWeight(op.input[4]);
        if (!scale || !bias || !mean || !var) return;
        const PbArgument *eps = op.find("epsilon");
        node = new OpNode(name, new BatchNormalizationOp(eps && eps->has_f ? eps->f : 1e-5f));
        node->exlinkUpperNode(in, scale, bias, mean, var);
        result(op.output[0], idims, node);
    } else if (op.type == "Relu") {
        node = new OpNode(name, new ReluOp());
        node->exlinkUpperNode(in);
        result(op.output[0], idims, node);
    } else if (op.type == "Sum") {
        TensorNode *rhs = op.input.size() > 1 ? tensor(op.input[1]) : nullptr;
        if (!rhs || rhs->getDims() != idims) {
            fail("Sum: needs two inputs of one shape");
            return;
        }
        node = new OpNode(name, new ElementAddOp());
        node->exlinkUpperNode(in, rhs);
        result(op.output[0], idims, node);
    } else if (op.type == "MaxPool" || op.type == "AveragePool") {
        if (idims.size() != 4) {
            fail(op.type + ": needs a 4-D input");
            return;
        }
        std::vector<size_t> k = pair(op, "kernel", 0), s = pair(op, "stride", 1), p = pads(op);
        if (k[0] == 0) {
            fail(op.type + ": no kernel argument");
            return;
        }
        node = op.type == "MaxPool" ? new OpNode(name, new MaxPoolOp(k, s, p)) : new OpNode(name, new AvgPoolOp(k, s, p));
        node->exlinkUpperNode(in);
        const std::vector<size_t> hw = outHW(idims[1], idims[2], k, s, p);
        result(op.output[0], {idims[0], hw[0], hw[1], idims[3]}, node);
    } else if (op.type == "FC") {
        auto wit = blobs_.find(op.input.size() > 1 ? op.input[1] : "");
        if (op.input.size() != 3 || wit == blobs_.end() || wit->second.shape.size() != 2) {
            fail("FC: needs a 2-D weight from the init net and a bias");
            return;
        }
        const Blob &w = wit->second;
        const size_t out = w.shape[0], k = w.shape[1];
        size_t flat = 1;
        for (size_t d = 1; d < idims.size(); d++) flat *= idims[d];
        if (flat != k) {
            fail("FC: the input flattens to " + std::to_string(flat) + ", the weight expects " + std::to_string(k));
            return;
        }
        // [out, in] -> [in, out]; a 4-D NHWC input flattens as (h, w, c) where Caffe2 counted (c, h, w)
        std::vector<float> v(w.values.size());
        if (idims.size() == 4) {
            const size_t H = idims[1], W = idims[2], Cc = idims[3];
            for (size_t o = 0; o < out; o++)
                for (size_t c = 0; c < Cc; c++)
                    for (size_t h = 0; h < H; h++)
                        for (size_t x = 0; x < W; x++)
                            v[((h * W + x) * Cc + c) * out + o] = w.values[o * k + (c * H + h) * W + x];
        } else {
            for (size_t o = 0; o < out; o++)
                for (size_t i = 0; i < k; i++) v[i * out + o] = w.values[o * k + i];
        }
        TensorNode *weight = weightNode(op.input[1], {k, out}, v), *bias = plainWeight(op.input[2]);
        if (!weight || !bias) return;
        node = new OpNode(name, new MatrixMatrixFCBiasOp());
        node->exlinkUpperNode(in, weight, bias);
        result(op.output[0], {idims[0], out}, node);
    } else if (op.type == "Softmax") {
        node = new OpNode(name, new MatrixSoftmaxOp());
        node->exlinkUpperNode(in);
        result(op.output[0], idims, node);
    } else {  // Dropout: the identity at inference; the mask the op class asks for is never read
        const PbArgument *ratio = op.find("ratio");
        auto *mask = new TensorNode(name + "_mask", newTensor(idims));
        mask->getTensor()->setTensorInit(TensorInitType::CONSTANT, 1.f);
        graph_->pushTensorNode(mask);
        node = new OpNode(name, new DropoutOp(ratio && ratio->has_f ? ratio->f : 0.5f));
        node->exlinkUpperNode(in, mask);
        result(op.output[0], idims, node);
    }
    graph_->pushOpNode(node);
}

}  // namespace swcb200
