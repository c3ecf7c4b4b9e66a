// Caffe2Import -- reads a Caffe2 model (predict_net.pb + init_net.pb) into an SWCompiler IRGraph without protobuf.
//
// The reference's importer (src/importer/Caffe2Importer.{h,cpp}, :176-471 for the operators, :473-557 for the
// weights) is generated-protobuf code and builds only where libprotobuf and protoc are installed.  This one parses
// the protobuf wire format of the three messages a model file holds (NetDef, OperatorDef, Argument; field numbers
// of src/importer/caffe2.proto:152-166, :210-246, :270-308) directly and builds the same kind of graph with the
// reference's public classes: the operator set is the reference's (Conv, SpatialBN, Relu, Sum, MaxPool,
// AveragePool, FC, Softmax, Dropout), activations are NHWC as everywhere in SWCompiler, weights arrive in Caffe2's
// layouts (filters oihw, FC weights [out, in] over (c, h, w)).
//
// One difference by design.  The reference keeps the weights as they come and inserts Transpose op nodes that re-lay
// them out (and the FC's 4-D input) on EVERY forward pass.  Here the re-layout happens ONCE, at import: a filter is
// written to its weight file as [o, h, w, i], an FC weight as [in, out] with its input index re-ordered from
// (c, h, w) to the (h, w, c) order an NHWC activation flattens to.  The forward pass then has no Transpose nodes;
// the numbers are the same (pure permutations).  Dropout is the identity at inference: its node stays in the
// graph and the generator prints it as an alias.
#pragma once

#include <cstdint>
#include <string>
#include <unordered_map>
#include <vector>

#include "graphIR/IRGraph.h"

namespace swcb200 {

// ---- the three messages, as plain structs
struct PbArgument {
    std::string name, s;
    float f = 0.f;
    int64_t i = 0;
    bool has_f = false, has_i = false, has_s = false;
    std::vector<float> floats;
    std::vector<int64_t> ints;
};
struct PbOperator {
    std::string type, name;
    std::vector<std::string> input, output;
    std::vector<PbArgument> arg;
    const PbArgument *find(const std::string &name) const;
};
struct PbNet {
    std::string name;
    std::vector<PbOperator> op;
    std::vector<std::string> external_input, external_output;
};

// Parses a serialized NetDef.  Unknown fields are skipped, packed and unpacked repeated scalars are both accepted.
// Returns false (and a message) on malformed input.
bool parseNetDef(const std::string &bytes, PbNet *net, std::string *error);

class Caffe2Import {
  public:
    // `inputs`: the tensor nodes the model does not define itself (the data), as in the reference's importer.
    // `weight_dir`: where the weight files go; the graph's tensors name them relative to it by `weight_prefix`.
    Caffe2Import(swc::IRGraph *graph, const std::string &predict_net_file, const std::string &init_net_file,
                 const std::vector<swc::TensorNode *> &inputs, const std::string &weight_dir,
                 const std::string &weight_prefix = "");

    bool ok() const { return error_.empty(); }
    const std::string &error() const { return error_; }
    swc::TensorNode *tensor(const std::string &blob) const;
    // the model's last output blob
    swc::TensorNode *output() const { return last_output_; }

  private:
    struct Blob {
        std::vector<size_t> shape;
        std::vector<float> values;  // GivenTensorFill
        bool constant = false;      // ConstantFill
        float fill = 0.f;
    };
    void loadWeights(const PbNet &init);
    void loadOperator(const PbOperator &op);
    swc::TensorNode *weightNode(const std::string &blob, const std::vector<size_t> &shape, const std::vector<float> &values);
    swc::TensorNode *plainWeight(const std::string &blob);
    swc::TensorNode *result(const std::string &blob, const std::vector<size_t> &dims, swc::OpNode *producer);
    bool fail(const std::string &why);

    swc::IRGraph *graph_;
    std::string weight_dir_, weight_prefix_, error_;
    std::unordered_map<std::string, Blob> blobs_;
    std::unordered_map<std::string, swc::TensorNode *> nodes_;
    std::unordered_map<std::string, int> op_names_;
    swc::TensorNode *last_output_ = nullptr;
};

}  // namespace swcb200
