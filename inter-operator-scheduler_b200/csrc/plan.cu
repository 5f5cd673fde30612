// Model -> launch list (see plan.h).
#include "plan.h"

#include <algorithm>
#include <cstring>
#include <map>

namespace ios {
namespace {

constexpr size_t kAlign = 256;

size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }
int round_up(int c, int m) { return (c + m - 1) / m * m; }

struct UserRef {
    int op;
    bool sole_value;   // the consumer reads this producer as a single-value term
};

class Lowering {
public:
    Lowering(Plan *plan, char *base, bool dry, int sm_count)
        : plan_(*plan), m_(plan->model), base_(base), dry_(dry), sms_(sm_count) {}

    void run() {
        const size_t n = m_.ops.size();
        plan_.steps.clear();
        plan_.convs.clear();
        plan_.tensors.assign(n, TensorRef());
        plan_.input_offsets.clear();
        placed_.assign(n, false);
        has_tensor_.assign(n, false);
        fused_relu_.assign(n, false);
        concat_in_.clear();
        users_.assign(n, {});
        for (size_t i = 0; i < n; ++i)
            for (const Term &term : m_.ops[i].inputs)
                for (const ValueRef &v : term) users_[v.node].push_back({int(i), term.size() == 1});

        cursor_ = 0;
        esize_ = plan_.options.bf16 ? 2 : 4;
        per16_ = 16 / esize_;                      // elements per 16 bytes: pixel pitches are multiples of it
        plan_.error_flag_offset = alloc(kAlign);
        // split-K arrival counters: one zero-initialised region, size known from the dry pass
        plan_.zero_begin = alloc(dry_ ? 0 : plan_.zero_bytes);
        counter_cursor_ = plan_.zero_begin;
        counter_end_ = plan_.zero_begin + (dry_ ? 0 : plan_.zero_bytes);
        counter_total_ = 0;
        // split-K workspaces: group j of every stage runs on stream j, one kernel after another, so the
        // convolutions of a group slot share one region, sized by the dry pass
        ws_need_.assign(plan_.group_workspace_bytes.size(), 0);
        ws_offset_.clear();
        if (!dry_)
            for (size_t bytes : plan_.group_workspace_bytes) ws_offset_.push_back(alloc(bytes));

        size_t in_floats = 0;
        for (int idx : m_.placeholders) {
            const Op &op = m_.ops[idx];
            const int pitch = round_up(op.C, per16_);
            const size_t off = alloc(size_t(m_.batch) * op.H * op.W * pitch * esize_);
            plan_.input_offsets.push_back(off);
            set_tensor(idx, window(off, op, pitch, 0, op.C));
            in_floats = std::max(in_floats, size_t(m_.batch) * op.C * op.H * op.W);
        }
        plan_.staging_in_offset = alloc(in_floats * sizeof(float));
        const Op &out = m_.ops[m_.output];
        plan_.staging_out_offset = alloc(size_t(m_.batch) * out.C * out.H * out.W * sizeof(float));
        plan_.input_round_tf32 = !m_.placeholders.empty() && rounds_for_consumers(m_.placeholders[0]);

        place_concats();

        plan_.max_groups = 1;
        if (dry_) plan_.workspace_bytes = 0;
        for (size_t s = 0; s < m_.stages.size(); ++s) {
            const auto &stage = m_.stages[s];
            plan_.max_groups = std::max(plan_.max_groups, int(stage.size()));
            for (size_t g = 0; g < stage.size(); ++g) {
                stage_ = int(s);
                group_ = int(g);
                width_ = int(stage.size());
                for (size_t k = 0; k < stage[g].size(); ++k) lower_op(stage[g][k], stage[g], k);
            }
        }
        plan_.launches_per_forward = int(plan_.steps.size());
        // Weights are read once per forward and do not fit the L2 together, so every convolution would meet its own
        // in DRAM: each tensor-core convolution asks the weights of the next one (in launch order) into L2 instead.
        {
            Step *previous = nullptr;
            for (Step &s : plan_.steps) {
                if (s.kind != StepKind::ConvTc) continue;
                s.tc.next_weights = nullptr;
                s.tc.next_weight_bytes = 0;
                if (previous && !plan_.options.no_weight_prefetch) {
                    size_t bytes = 0;
                    for (const ConvSlot &c : plan_.convs)
                        if (c.op == s.op) bytes = c.weight_bytes;
                    previous->tc.next_weights = s.tc.weight_packed;
                    previous->tc.next_weight_bytes = unsigned(std::min<size_t>(bytes, size_t(16) << 20) & ~size_t(127));
                }
                previous = &s;
            }
        }
        if (dry_) {
            plan_.zero_bytes = counter_total_;
            plan_.group_workspace_bytes = ws_need_;
            size_t ws_total = 0;
            for (size_t bytes : ws_need_) ws_total += align_up(bytes, kAlign) + kAlign;
            plan_.workspace_bytes = ws_total;
            plan_.arena_bytes = align_up(cursor_ + counter_total_ + ws_total + kAlign, 4096);
        }
    }

private:
    Plan &plan_;
    Model &m_;
    char *base_;
    bool dry_;
    int sms_;
    size_t cursor_ = 0, counter_cursor_ = 0, counter_end_ = 0, counter_total_ = 0;
    std::vector<size_t> ws_need_, ws_offset_;     // split-K workspace per group slot: bytes needed (dry pass), arena offset
    int stage_ = 0, group_ = 0, width_ = 1;
    int esize_ = 4, per16_ = 4;
    std::vector<bool> placed_, has_tensor_;
    std::vector<std::vector<UserRef>> users_;
    std::map<int, TensorRef> concat_in_;          // assembled-input buffer of multi-term Conv / Pool ops
    std::map<int, std::vector<bool>> term_placed_;
    std::vector<bool> fused_relu_;                // Relu ops folded into the consumer's read

    size_t alloc(size_t bytes) {
        cursor_ = align_up(cursor_, kAlign);
        const size_t off = cursor_;
        cursor_ += bytes;
        return off;
    }
    float *at(size_t off) const { return reinterpret_cast<float *>(base_ + off); }

    TensorRef window(size_t off, const Op &op, int pitch, int c0, int c) const {
        TensorRef t;
        t.esize = esize_;
        t.ptr = reinterpret_cast<char *>(at(off)) + size_t(c0) * esize_;
        t.N = m_.batch;
        t.H = op.H;
        t.W = op.W;
        t.C = c;
        t.pitch = pitch;
        return t;
    }
    static TensorRef slice(const TensorRef &whole, int begin, int end) {
        TensorRef t = whole.shifted(begin);
        t.C = end - begin;
        return t;
    }
    void set_tensor(int idx, const TensorRef &t) {
        plan_.tensors[idx] = t;
        has_tensor_[idx] = true;
    }
    TensorRef fresh(const Op &op, int channels) {
        const int pitch = round_up(channels, per16_);
        const size_t off = alloc(size_t(m_.batch) * op.H * op.W * pitch * esize_);
        return window(off, op, pitch, 0, channels);
    }

    // ---- which convolutions will run on the tensor cores (by geometry; view alignment is checked later)
    // A convolution over at most 4 input channels (a network's stem) is bound by the bytes it writes; from
    // some 150 000 output pixels on (Inception-v3 at batch 7) it is faster on CUDA cores
    // (launch_conv_direct's form for few input channels: measured 1.5x at batch 64) whatever the precision.
    // Below that the tensor-core kernel's split over the taps wins.
    bool few_channels(const Op &op) const {
        return !plan_.options.no_stem_kernel && op.groups == 1 && op.inC <= 4 && op.C % 4 == 0 &&
               size_t(op.kh) * op.kw * op.inC * op.C * sizeof(float) <= 96 * 1024 &&
               long(m_.batch) * op.H * op.W >= 150000;
    }
    bool tc_candidate(const Op &op) const {
        return op.kind == OpKind::Conv && op.groups == 1 && (plan_.options.tf32 || plan_.options.bf16) && plan_.options.allow_tc &&
               op.sh <= 8 && op.sw <= 8 && !few_channels(op);
    }
    // Round a tensor to TF32 when it is stored?  Only if every reader is a tensor-core convolution
    // that takes it unchanged, and it is not the tensor handed back to the caller.
    // Identity operators hand their single-value terms on unchanged, so the test looks through them.
    bool rounds_for_consumers(int idx) const {
        if (!plan_.options.tf32 || plan_.options.three_pass || plan_.options.bf16 || idx == m_.output || users_[idx].empty())
            return false;
        for (const UserRef &u : users_[idx]) {
            const Op &c = m_.ops[u.op];
            if (!u.sole_value || !c.scheduled) return false;
            if (c.kind == OpKind::Identity) {
                if (!rounds_for_consumers(u.op)) return false;
            } else if (!tc_candidate(c)) {
                return false;
            }
        }
        return true;
    }

    // ---- concat by placement -----------------------------------------------------------------
    bool placeable_producer(const Op &p) const {
        if (!p.scheduled) return false;
        switch (p.kind) {
            case OpKind::Conv: case OpKind::Pool: case OpKind::Relu: case OpKind::Activation: case OpKind::Element:
                return true;
            case OpKind::Identity:
                return p.inputs.size() > 1 || p.inputs[0].size() > 1;   // it materialises something
            default:
                return false;
        }
    }
    void place_concats() {
        term_placed_.clear();
        for (int x = int(m_.ops.size()) - 1; x >= 0; --x) {
            const Op &op = m_.ops[x];
            if (!op.scheduled || op.inputs.size() < 2) continue;
            if (op.kind != OpKind::Identity && op.kind != OpKind::Conv && op.kind != OpKind::Pool) continue;
            TensorRef buf;
            if (op.kind == OpKind::Identity && has_tensor_[x]) {
                buf = plan_.tensors[x];                       // this concat is itself a member of a later concat
            } else {
                Op shape = op;
                shape.H = op.inH;
                shape.W = op.inW;
                buf = fresh(shape, op.inC);
            }
            if (op.kind == OpKind::Identity) set_tensor(x, buf);
            else concat_in_[x] = buf;
            std::vector<bool> flags(op.inputs.size(), false);
            int c_off = 0;
            for (size_t t = 0; t < op.inputs.size(); ++t) {
                const Term &term = op.inputs[t];
                const int tc = term[0].end - term[0].begin;
                if (term.size() == 1) {
                    const ValueRef &v = term[0];
                    const Op &p = m_.ops[v.node];
                    const bool whole = v.begin == 0 && v.end == p.C;
                    const bool aligned = (c_off % per16_ == 0 && (reinterpret_cast<uintptr_t>(buf.ptr) & 15) == 0) ||
                                         users_[v.node].size() == 1;
                    if (whole && !has_tensor_[v.node] && placeable_producer(p) && aligned) {
                        set_tensor(v.node, slice(buf, c_off, c_off + tc));
                        placed_[v.node] = true;
                        flags[t] = true;
                    }
                }
                c_off += tc;
            }
            term_placed_[x] = flags;
        }
    }

    // ---- launches ----------------------------------------------------------------------------
    Step &push(StepKind kind, int op) {
        Step s;
        std::memset(static_cast<void *>(&s.sum), 0, sizeof s.sum);
        s.kind = kind;
        s.stage = stage_;
        s.group = group_;
        s.op = op;
        plan_.steps.push_back(s);
        return plan_.steps.back();
    }

    // dst = act(sum or product of the values of `term`); chains launches of at most 8 inputs
    void emit_term(int op_idx, const Term &term, const TensorRef &dst, Act act, bool mul, bool round_out) {
        size_t done = 0;
        bool first = true;
        while (done < term.size()) {
            Step &s = push(StepKind::SumAct, op_idx);
            SumActParams &p = s.sum;
            int k = 0;
            bool vec = dst.vec4();
            if (!first) {                       // carry the partial result
                p.in[k] = dst.ptr;
                p.in_pitch[k] = dst.pitch;
                ++k;
            }
            while (k < kMaxSumInputs && done < term.size()) {
                const ValueRef &v = term[done++];
                const TensorRef src = slice(plan_.tensors[v.node], v.begin, v.end);
                p.in[k] = src.ptr;
                p.in_pitch[k] = src.pitch;
                vec = vec && src.vec4();
                ++k;
            }
            const bool last = done == term.size();
            p.k = k;
            p.out = dst.ptr;
            p.out_pitch = dst.pitch;
            p.esize = esize_;
            p.C = dst.C;
            p.pixels = dst.pixels();
            p.act = last ? int(act) : 0;
            p.mul = mul ? 1 : 0;
            p.round_out = (last && round_out) ? 1 : 0;
            s.vec4 = vec;
            first = false;
        }
    }

    // Assembled input of a Conv / Pool.
    TensorRef input_of(int idx, bool round_tmp) {
        const Op &op = m_.ops[idx];
        if (op.inputs.size() == 1) {
            const Term &term = op.inputs[0];
            if (term.size() == 1) return slice(plan_.tensors[term[0].node], term[0].begin, term[0].end);
            Op shape = op;
            shape.H = op.inH;
            shape.W = op.inW;
            TensorRef tmp = fresh(shape, op.inC);
            emit_term(idx, term, tmp, Act::Identity, false, round_tmp);
            return tmp;
        }
        const TensorRef buf = concat_in_.at(idx);
        fill_unplaced_terms(idx, buf, Act::Identity, false, round_tmp);
        return buf;
    }
    void fill_unplaced_terms(int idx, const TensorRef &buf, Act act, bool mul, bool round_out) {
        const Op &op = m_.ops[idx];
        auto it = term_placed_.find(idx);
        int c_off = 0;
        for (size_t t = 0; t < op.inputs.size(); ++t) {
            const int tc = op.inputs[t][0].end - op.inputs[t][0].begin;
            const bool skip = it != term_placed_.end() && it->second[t];
            if (!skip) emit_term(idx, op.inputs[t], slice(buf, c_off, c_off + tc), act, mul, round_out);
            c_off += tc;
        }
    }

    TensorRef output_of(int idx) {
        if (!has_tensor_[idx]) set_tensor(idx, fresh(m_.ops[idx], m_.ops[idx].C));
        return plan_.tensors[idx];
    }

    void lower_op(int idx, const std::vector<int> &group, size_t pos) {
        Op &op = m_.ops[idx];
        const bool round_out = rounds_for_consumers(idx);
        switch (op.kind) {
            case OpKind::Identity:
                if (op.inputs.size() == 1 && op.inputs[0].size() == 1) {
                    const ValueRef &v = op.inputs[0][0];
                    if (!has_tensor_[idx]) {
                        set_tensor(idx, slice(plan_.tensors[v.node], v.begin, v.end));   // alias, no launch
                        return;
                    }
                }
                if (op.inputs.size() > 1) {
                    fill_unplaced_terms(idx, plan_.tensors[idx], Act::Identity, false, round_out);
                    return;
                }
                emit_term(idx, op.inputs[0], output_of(idx), Act::Identity, false, round_out);
                return;
            case OpKind::Relu:
            case OpKind::Activation:
            case OpKind::Element: {
                // A lone ReLU whose only reader is the depthwise / CUDA-core convolution launched right
                // after it in the same group is folded into that convolution's read.
                if (op.kind == OpKind::Relu && can_fold_relu(idx, group, pos)) {
                    const ValueRef &v = op.inputs[0][0];
                    set_tensor(idx, slice(plan_.tensors[v.node], v.begin, v.end));
                    fused_relu_[idx] = true;
                    return;
                }
                const TensorRef out = output_of(idx);
                int c_off = 0;
                for (const Term &term : op.inputs) {
                    const int tc = term[0].end - term[0].begin;
                    emit_term(idx, term, slice(out, c_off, c_off + tc), op.act, op.elem_mul, round_out);
                    c_off += tc;
                }
                return;
            }
            case OpKind::Pool: {
                const TensorRef in = input_of(idx, false);
                Step &s = push(StepKind::Pool, idx);
                s.pool.in = in;
                s.pool.out = output_of(idx);
                s.pool.kh = op.kh; s.pool.kw = op.kw; s.pool.sh = op.sh; s.pool.sw = op.sw;
                s.pool.ph = op.ph; s.pool.pw = op.pw;
                s.pool.is_max = op.pool_max ? 1 : 0;
                s.pool.round_out = round_out ? 1 : 0;
                return;
            }
            case OpKind::Conv:
                lower_conv(idx, round_out);
                return;
            default:
                throw GraphError("operator '" + op.name + "' cannot be scheduled");
        }
    }

    bool direct_kind(const Op &c) const {
        return c.kind == OpKind::Conv && !(tc_candidate(c));
    }
    bool can_fold_relu(int idx, const std::vector<int> &group, size_t pos) const {
        const Op &op = m_.ops[idx];
        if (op.inputs.size() != 1 || op.inputs[0].size() != 1) return false;
        if (users_[idx].size() != 1 || has_tensor_[idx] || idx == m_.output) return false;
        if (pos + 1 >= group.size() || group[pos + 1] != users_[idx][0].op) return false;
        const Op &c = m_.ops[users_[idx][0].op];
        return direct_kind(c) && c.inputs.size() == 1 && c.inputs[0].size() == 1 &&
               c.inputs[0][0].begin == 0 && c.inputs[0][0].end == op.C;
    }

    void lower_conv(int idx, bool round_out) {
        const Op &op = m_.ops[idx];
        const bool tc_wanted = tc_candidate(op);
        bool pre_relu = false;
        if (op.inputs.size() == 1 && op.inputs[0].size() == 1) {
            const int src = op.inputs[0][0].node;
            pre_relu = src < int(fused_relu_.size()) && fused_relu_[src];
        }
        const TensorRef in = input_of(idx, tc_wanted);
        const TensorRef out = output_of(idx);
        ConvGeom g;
        g.N = m_.batch; g.Cin = op.inC; g.H = op.inH; g.W = op.inW;
        g.Cout = op.C; g.OH = op.H; g.OW = op.W;
        g.kh = op.kh; g.kw = op.kw; g.sh = op.sh; g.sw = op.sw; g.ph = op.ph; g.pw = op.pw;
        g.groups = op.groups;
        g.act = int(op.act);
        g.pre_relu = pre_relu ? 1 : 0;
        g.round_out = round_out ? 1 : 0;

        ConvSlot slot;
        slot.op = idx;
        slot.geom = g;
        std::memset(static_cast<void *>(&slot.tcplan), 0, sizeof slot.tcplan);
        const bool depthwise = op.groups > 1 && op.groups == op.inC && op.groups == op.C;
        if (depthwise) {
            slot.impl = StepKind::ConvDepthwise;
            slot.weight_bytes = size_t(op.kh) * op.kw * ((op.C + 3) / 4 * 4) * sizeof(float);   // rows padded to 4
        } else if (tc_wanted && conv_tc_supported(in, g)) {
            slot.impl = StepKind::ConvTc;
            slot.tcplan.no_persistent = plan_.options.no_persistent ? 1 : 0;
            slot.tcplan.no_push = plan_.options.no_cluster_push ? 1 : 0;
            slot.tcplan.no_dual = plan_.options.no_dual_issue ? 1 : 0;
            slot.tcplan.no_half_rows = plan_.options.no_half_rows ? 1 : 0;
            conv_tc_choose(g, sms_, width_, plan_.options.three_pass, &slot.tcplan, plan_.options.force_bn, plan_.options.bf16,
                           !plan_.options.no_im2col);
            if (plan_.options.force_split_k > 0) conv_tc_set_split(&slot.tcplan, plan_.options.force_split_k);
            slot.tcplan.no_patch = plan_.options.no_patch ? 1 : 0;
            slot.tcplan.patch_all = plan_.options.patch_all ? 1 : 0;
            slot.tcplan.max_issuers = plan_.options.patch_issuers;
            slot.tcplan.patch_bulk_store = plan_.options.patch_bulk_store ? 1 : 0;
            conv_tc_patch_consider(g, sms_, &slot.tcplan);
            slot.tcplan.pdl = plan_.options.pdl ? 1 : 0;
            slot.tcplan.max_producers = plan_.options.producers;
            if (plan_.options.force_stages > 0 && !slot.tcplan.persistent && !slot.tcplan.patch && !slot.tcplan.push) {   // testing aid: shallower pipeline
                ConvTcPlan &q = slot.tcplan;
                const size_t stage_bytes = (q.smem_bytes - 24 * q.stages - 64 - 1024) / q.stages;   // (whatever the row width)
                const int stages = std::max(2, std::min(q.stages, plan_.options.force_stages));
                if (size_t(stages) * stage_bytes >= size_t(128) * (q.bn + 4) * 4 && size_t(stages) * stage_bytes >= size_t(q.bn / 32) * 16384) {
                    q.stages = stages;
                    q.smem_bytes = size_t(stages) * stage_bytes + 24 * stages + 64 + 1024;
                }
            }
            slot.weight_bytes = conv_tc_packed_bytes(g, slot.tcplan);
        } else {
            slot.impl = StepKind::ConvDirect;
            slot.weight_bytes = size_t(op.kh) * op.kw * (op.inC / op.groups) * op.C * sizeof(float);
        }
        slot.weight_offset = alloc(slot.weight_bytes);
        slot.bias_offset = alloc(size_t(op.C) * sizeof(float));

        Step &s = push(slot.impl, idx);
        if (slot.impl == StepKind::ConvTc) {
            s.tc.in = in;
            s.tc.out = out;
            s.tc.weight_packed = at(slot.weight_offset);
            s.tc.bias = at(slot.bias_offset);
            s.tc.g = g;
            s.tc.error_flag = reinterpret_cast<int *>(at(plan_.error_flag_offset));
            s.tc.workspace = nullptr;
            s.tc.counters = nullptr;
            s.tc.next_weights = nullptr;
            s.tc.next_weight_bytes = 0;
            s.tc.timeline = plan_.options.timeline ? reinterpret_cast<long long *>(at(plan_.error_flag_offset) + 16) : nullptr;
            if (slot.tcplan.split_k > 1) {
                if (dry_) {
                    if (ws_need_.size() <= size_t(group_)) ws_need_.resize(group_ + 1, 0);
                    ws_need_[group_] = std::max(ws_need_[group_], slot.tcplan.workspace_bytes);
                } else if (slot.tcplan.workspace_bytes > 0) {
                    if (size_t(group_) >= ws_offset_.size() || plan_.group_workspace_bytes[group_] < slot.tcplan.workspace_bytes)
                        throw std::runtime_error("internal: split-K workspace of a group slot is too small");
                    s.tc.workspace = reinterpret_cast<float *>(at(ws_offset_[group_]));
                }
                counter_total_ += align_up(slot.tcplan.counter_bytes, 16);
                if (!dry_) {
                    s.tc.counters = reinterpret_cast<unsigned int *>(at(counter_cursor_));
                    counter_cursor_ += align_up(slot.tcplan.counter_bytes, 16);
                    if (counter_cursor_ > counter_end_) throw std::runtime_error("internal: split-K counter region overflow");
                }
            }
            if (!dry_) {
                const char *err = conv_tc_encode(s.tc, &slot.tcplan);
                if (err) throw std::runtime_error(err);
                if (plan_.options.no_bulk_store) slot.tcplan.tma_store = 0;   // testing aid
            }
            s.tcplan = slot.tcplan;
        } else {
            s.direct.in = in;
            s.direct.out = out;
            s.direct.weight = at(slot.weight_offset);
            s.direct.bias = at(slot.bias_offset);
            s.direct.g = g;
        }
        plan_.convs.push_back(slot);
    }
};

}  // namespace

void plan_layout(Plan *plan, int sm_count) {
    // a 1 MiB-aligned stand-in base keeps every alignment decision identical to the bound pass
    Lowering pass(plan, reinterpret_cast<char *>(uintptr_t(1) << 20), true, sm_count);
    pass.run();
}

void plan_bind(Plan *plan, char *arena_base, int sm_count) {
    Lowering pass(plan, arena_base, false, sm_count);
    pass.run();
}

}  // namespace ios
