// Host-side model of a scheduled IOS graph: operators in topological order with their input
// algebra (concat over terms of sums over channel slices) and the stage / group schedule.
//
// Built from the JSON wire format of python/ios/ir.py (Graph / Block / Node.export_config) or,
// for the stage profiler, from a list of groups of node configs plus an input-shape map
// (python/ios/contrib/ios_runtime.py:80-99).  Replaces Graph::init_graph / init_block / init_stage /
// add_node of the reference runtime (src/ios/ios_runtime.cu:1118-1240) without its fixed-size
// tables: compound Sequential operators are flattened into their inner operators, shapes are
// always re-inferred (a config's output_shape may be null), and every structural problem raises
// GraphError instead of terminating the process.
#pragma once
#include <map>
#include <stdexcept>
#include <string>
#include <vector>

#include "json.h"

namespace ios {

struct GraphError : std::runtime_error {
    explicit GraphError(const std::string &what) : std::runtime_error(what) {}
};

enum class OpKind { Placeholder, Conv, Pool, Identity, Relu, Activation, Element };
enum class Act : int { Identity = 0, Relu = 1, Sigmoid = 2, Tanh = 3 };

struct ValueRef {
    int node;    // index into Model::ops
    int begin;   // channel slice [begin, end) of that operator's output
    int end;
};
using Term = std::vector<ValueRef>;

struct Op {
    OpKind kind = OpKind::Placeholder;
    std::string name;
    std::vector<Term> inputs;
    int C = 0, H = 0, W = 0;         // output shape (per image)
    int inC = 0, inH = 0, inW = 0;   // shape of the assembled input
    // convolution / pooling geometry
    int kh = 1, kw = 1, sh = 1, sw = 1, ph = 0, pw = 0, groups = 1;
    Act act = Act::Identity;         // conv epilogue, Relu, Activation
    bool pool_max = false;
    bool elem_mul = false;
    bool inplace = false;
    bool scheduled = false;
    int num_users = 0;               // value references from other operators
};

struct Model {
    int batch = 1;
    std::vector<Op> ops;                                  // producers before consumers
    std::map<std::string, int> by_name;                   // a Sequential's name maps to its last inner op
    std::vector<std::vector<std::vector<int>>> stages;    // stage -> group -> op indices, in launch order
    std::vector<int> placeholders;
    int output = -1;                                      // op whose tensor graph_inference returns
    bool output_is_single_group = true;                   // the last stage has exactly one group

    double conv_flops() const;                            // 2 * MACs of every scheduled convolution, whole batch
};

Model model_from_graph(const Json &graph, int batch);
Model model_from_block(const Json &block, int batch);
Model model_from_stage(const Json &stage, const Json &inputs, int batch);

}  // namespace ios
