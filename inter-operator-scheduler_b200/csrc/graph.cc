// JSON -> Model (see graph.h).
#include "graph.h"

#include <set>

namespace ios {
namespace {

constexpr int kMaxGroupsPerStage = 64;   // the reference stops at 10 (src/ios/ios_runtime.cu:46)

struct Builder {
    Model model;
    std::map<std::string, std::vector<int>> unit_ops;   // schedule-unit name -> ops it launches, in order

    static int int_at(const Json &cfg, const char *key, size_t i) {
        const Json &arr = cfg.at(key);
        if (!arr.is_array() || arr.size() <= i) throw GraphError(std::string("field '") + key + "' needs two entries");
        return arr.at(i).as_int();
    }

    int add_placeholder(const std::string &name, int c, int h, int w) {
        if (c <= 0 || h <= 0 || w <= 0) throw GraphError("placeholder '" + name + "' has a non-positive shape");
        Op op;
        op.kind = OpKind::Placeholder;
        op.name = name;
        op.C = c;
        op.H = h;
        op.W = w;
        op.scheduled = true;
        int idx = static_cast<int>(model.ops.size());
        model.ops.push_back(op);
        model.by_name[name] = idx;
        model.placeholders.push_back(idx);
        return idx;
    }

    int add_placeholder(const Json &cfg) {
        const Json &shape = cfg.at("output_shape");
        if (!shape.is_array() || shape.size() != 3) throw GraphError("placeholder output_shape must be [C, H, W]");
        return add_placeholder(cfg.at("name").as_string(), shape.at(0).as_int(), shape.at(1).as_int(),
                               shape.at(2).as_int());
    }

    void read_inputs(Op &op, const Json &inputs) {
        if (!inputs.is_array() || inputs.size() == 0)
            throw GraphError("operator '" + op.name + "' has no inputs");
        int total_c = 0;
        for (size_t t = 0; t < inputs.size(); ++t) {
            const Json &term_cfg = inputs.at(t);
            if (!term_cfg.is_array() || term_cfg.size() == 0)
                throw GraphError("operator '" + op.name + "' has an empty term");
            Term term;
            int tc = 0, th = 0, tw = 0;
            for (size_t v = 0; v < term_cfg.size(); ++v) {
                const Json &val = term_cfg.at(v);
                if (!val.is_array() || val.size() != 3)
                    throw GraphError("a value of '" + op.name + "' is not [name, begin, end]");
                const std::string &src = val.at(0).as_string();
                auto it = model.by_name.find(src);
                if (it == model.by_name.end())
                    throw GraphError("operator '" + op.name + "' reads unknown node '" + src + "'");
                ValueRef ref{it->second, val.at(1).as_int(), val.at(2).as_int()};
                const Op &prod = model.ops[ref.node];
                if (ref.begin < 0 || ref.end > prod.C || ref.begin >= ref.end)
                    throw GraphError("operator '" + op.name + "' slices '" + src + "' outside its channels");
                int c = ref.end - ref.begin;
                if (v == 0) {
                    tc = c;
                    th = prod.H;
                    tw = prod.W;
                } else if (c != tc || prod.H != th || prod.W != tw) {
                    throw GraphError("the values of a term of '" + op.name + "' differ in shape");
                }
                term.push_back(ref);
            }
            if (t == 0) {
                op.inH = th;
                op.inW = tw;
            } else if (th != op.inH || tw != op.inW) {
                throw GraphError("the terms of '" + op.name + "' differ in resolution");
            }
            total_c += tc;
            op.inputs.push_back(std::move(term));
        }
        op.inC = total_c;
    }

    static int out_extent(int in, int k, int p, int s, const std::string &name) {
        if (s <= 0 || k <= 0 || p < 0) throw GraphError("operator '" + name + "' has a bad kernel/stride/padding");
        int span = in - k + 2 * p;
        if (span < 0) throw GraphError("operator '" + name + "' has a window larger than its padded input");
        return 1 + span / s;
    }

    static Act act_from(const std::string &s, const std::string &name) {
        if (s == "identity") return Act::Identity;
        if (s == "relu") return Act::Relu;
        if (s == "sigmoid") return Act::Sigmoid;
        if (s == "tanh") return Act::Tanh;
        throw GraphError("operator '" + name + "' has unknown activation '" + s + "'");
    }

    int push(Op &&op) {
        if (model.by_name.count(op.name)) throw GraphError("duplicate node name '" + op.name + "'");
        for (const Term &term : op.inputs)
            for (const ValueRef &v : term) model.ops[v.node].num_users++;
        int idx = static_cast<int>(model.ops.size());
        model.by_name[op.name] = idx;
        model.ops.push_back(std::move(op));
        return idx;
    }

    // Adds one node config; appends the ops it launches to `launch`; returns the op holding its output.
    int add_node(const Json &cfg, std::vector<int> &launch) {
        if (!cfg.is_object()) throw GraphError("a node config is not an object");
        const std::string &type = cfg.at("type").as_string();
        const std::string &name = cfg.at("name").as_string();
        if (type == "sequential") {
            const Json &nodes = cfg.at("nodes");
            if (!nodes.is_array() || nodes.size() == 0) throw GraphError("sequential '" + name + "' is empty");
            int last = -1;
            for (size_t i = 0; i < nodes.size(); ++i) last = add_node(nodes.at(i), launch);
            if (model.by_name.count(name)) throw GraphError("duplicate node name '" + name + "'");
            model.by_name[name] = last;
            return last;
        }
        Op op;
        op.name = name;
        read_inputs(op, cfg.at("inputs"));
        op.C = op.inC;
        op.H = op.inH;
        op.W = op.inW;
        if (type == "conv") {
            op.kind = OpKind::Conv;
            op.C = cfg.at("out_channels").as_int();
            op.kh = int_at(cfg, "kernel", 0);
            op.kw = int_at(cfg, "kernel", 1);
            op.sh = int_at(cfg, "stride", 0);
            op.sw = int_at(cfg, "stride", 1);
            op.ph = int_at(cfg, "padding", 0);
            op.pw = int_at(cfg, "padding", 1);
            op.groups = cfg.at("groups").as_int();
            op.act = act_from(cfg.at("act").as_string(), name);
            if (op.C <= 0 || op.groups <= 0 || op.inC % op.groups || op.C % op.groups)
                throw GraphError("conv '" + name + "': groups must divide input and output channels");
            op.H = out_extent(op.inH, op.kh, op.ph, op.sh, name);
            op.W = out_extent(op.inW, op.kw, op.pw, op.sw, name);
        } else if (type == "pool") {
            op.kind = OpKind::Pool;
            const std::string &pt = cfg.at("pool_type").as_string();
            op.pool_max = pt.find("max") != std::string::npos;
            if (!op.pool_max && pt.find("avg") == std::string::npos)
                throw GraphError("pool '" + name + "' has unknown pool_type '" + pt + "'");
            if (pt.find("global") != std::string::npos) {
                op.kh = op.inH;
                op.kw = op.inW;
            } else {
                op.kh = int_at(cfg, "kernel", 0);
                op.kw = int_at(cfg, "kernel", 1);
                op.sh = int_at(cfg, "stride", 0);
                op.sw = int_at(cfg, "stride", 1);
                op.ph = int_at(cfg, "padding", 0);
                op.pw = int_at(cfg, "padding", 1);
            }
            op.H = out_extent(op.inH, op.kh, op.ph, op.sh, name);
            op.W = out_extent(op.inW, op.kw, op.pw, op.sw, name);
        } else if (type == "identity") {
            op.kind = OpKind::Identity;
        } else if (type == "relu") {
            op.kind = OpKind::Relu;
            op.act = Act::Relu;
        } else if (type == "activation") {
            op.kind = OpKind::Activation;
            op.act = act_from(cfg.at("act_type").as_string(), name);
            if (op.act == Act::Identity) throw GraphError("activation '" + name + "' needs relu, tanh or sigmoid");
            const Json *inplace = cfg.find("inplace");
            op.inplace = inplace && !inplace->is_null() && inplace->as_bool();
        } else if (type == "element") {
            op.kind = OpKind::Element;
            const std::string &ot = cfg.at("op_type").as_string();
            if (ot != "add" && ot != "mul") throw GraphError("element '" + name + "' has unknown op_type '" + ot + "'");
            op.elem_mul = ot == "mul";
        } else {
            throw GraphError("unsupported node type '" + type + "'");
        }
        int idx = push(std::move(op));
        launch.push_back(idx);
        return idx;
    }

    void add_unit(const Json &cfg) {
        std::vector<int> launch;
        add_node(cfg, launch);
        unit_ops[cfg.at("name").as_string()] = std::move(launch);
    }

    void schedule_group(std::vector<int> &group_out, const std::vector<int> &launch,
                        const std::set<int> &done_before_stage, std::set<int> &done_in_group) {
        for (int idx : launch) {
            Op &op = model.ops[idx];
            if (op.scheduled) throw GraphError("operator '" + op.name + "' is scheduled twice");
            for (const Term &term : op.inputs)
                for (const ValueRef &v : term) {
                    const Op &prod = model.ops[v.node];
                    if (prod.kind == OpKind::Placeholder) continue;
                    if (!done_before_stage.count(v.node) && !done_in_group.count(v.node))
                        throw GraphError("operator '" + op.name + "' is scheduled before its producer '" +
                                         prod.name + "' finishes");
                }
            op.scheduled = true;
            done_in_group.insert(idx);
            group_out.push_back(idx);
        }
    }

    void add_stages(const Json &stages) {
        if (!stages.is_array()) throw GraphError("'stages' is missing: call sequential_schedule() or optimize() first");
        std::set<int> done;
        for (const auto &stage : model.stages)
            for (const auto &group : stage) done.insert(group.begin(), group.end());
        for (size_t s = 0; s < stages.size(); ++s) {
            const Json &stage_cfg = stages.at(s);
            if (!stage_cfg.is_array() || stage_cfg.size() == 0) throw GraphError("a stage has no groups");
            if (stage_cfg.size() > static_cast<size_t>(kMaxGroupsPerStage))
                throw GraphError("limit: a stage has more than " + std::to_string(kMaxGroupsPerStage) + " groups");
            std::vector<std::vector<int>> stage;
            std::set<int> done_in_stage;
            for (size_t g = 0; g < stage_cfg.size(); ++g) {
                const Json &group_cfg = stage_cfg.at(g);
                if (!group_cfg.is_array() || group_cfg.size() == 0) throw GraphError("a group has no operators");
                std::vector<int> group;
                std::set<int> done_in_group;
                for (size_t k = 0; k < group_cfg.size(); ++k) {
                    const std::string &unit = group_cfg.at(k).as_string();
                    auto it = unit_ops.find(unit);
                    if (it == unit_ops.end()) throw GraphError("the schedule names unknown operator '" + unit + "'");
                    schedule_group(group, it->second, done, done_in_group);
                }
                done_in_stage.insert(done_in_group.begin(), done_in_group.end());
                stage.push_back(std::move(group));
            }
            done.insert(done_in_stage.begin(), done_in_stage.end());
            model.stages.push_back(std::move(stage));
        }
    }

    void add_block(const Json &block) {
        const Json &inner = block.at("inner_nodes");
        if (!inner.is_array()) throw GraphError("'inner_nodes' must be an array");
        for (size_t i = 0; i < inner.size(); ++i) add_unit(inner.at(i));
        add_unit(block.at("exit_node"));
        add_stages(block.at("stages"));
    }

    Model finish() {
        if (model.stages.empty()) throw GraphError("the schedule is empty");
        const auto &last = model.stages.back();
        model.output_is_single_group = last.size() == 1;
        model.output = last[0].back();
        return std::move(model);
    }
};

void check_batch(int batch) {
    if (batch <= 0) throw GraphError("batch size must be positive");
}

}  // namespace

double Model::conv_flops() const {
    double total = 0.0;
    for (const auto &stage : stages)
        for (const auto &group : stage)
            for (int idx : group) {
                const Op &op = ops[idx];
                if (op.kind != OpKind::Conv) continue;
                total += 2.0 * op.C * op.H * op.W * (double(op.kh) * op.kw * (op.inC / op.groups));
            }
    return total * batch;
}

Model model_from_graph(const Json &graph, int batch) {
    check_batch(batch);
    Builder b;
    b.model.batch = batch;
    b.add_placeholder(graph.at("input"));
    const Json &blocks = graph.at("blocks");
    if (!blocks.is_array() || blocks.size() == 0) throw GraphError("the graph has no blocks");
    for (size_t i = 0; i < blocks.size(); ++i) b.add_block(blocks.at(i));
    return b.finish();
}

Model model_from_block(const Json &block, int batch) {
    check_batch(batch);
    Builder b;
    b.model.batch = batch;
    b.add_placeholder(block.at("enter_node"));
    b.add_block(block);
    return b.finish();
}

Model model_from_stage(const Json &stage, const Json &inputs, int batch) {
    check_batch(batch);
    Builder b;
    b.model.batch = batch;
    if (!inputs.is_object()) throw GraphError("the stage input map must be an object {name: [C, H, W]}");
    for (const auto &m : inputs.members) {
        if (!m.second.is_array() || m.second.size() != 3) throw GraphError("stage input '" + m.first + "' needs [C, H, W]");
        b.add_placeholder(m.first, m.second.at(0).as_int(), m.second.at(1).as_int(), m.second.at(2).as_int());
    }
    if (!stage.is_array() || stage.size() == 0) throw GraphError("the stage has no groups");
    if (stage.size() > static_cast<size_t>(kMaxGroupsPerStage))
        throw GraphError("limit: a stage has more than " + std::to_string(kMaxGroupsPerStage) + " groups");
    std::vector<std::vector<int>> groups;
    std::set<int> none;
    for (size_t g = 0; g < stage.size(); ++g) {
        const Json &group_cfg = stage.at(g);
        if (!group_cfg.is_array() || group_cfg.size() == 0) throw GraphError("a group has no operators");
        std::vector<int> group;
        std::set<int> done_in_group;
        for (size_t k = 0; k < group_cfg.size(); ++k) {
            std::vector<int> launch;
            b.add_node(group_cfg.at(k), launch);
            b.schedule_group(group, launch, none, done_in_group);
        }
        groups.push_back(std::move(group));
    }
    b.model.stages.push_back(std::move(groups));
    return b.finish();
}

}  // namespace ios
