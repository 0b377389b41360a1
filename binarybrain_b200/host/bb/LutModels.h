// bb::DifferentiableLutN<6>, bb::StochasticLutN<6>, bb::BinaryLutN<6>, bb::StochasticBatchNormalization,
// bb::OptimizerAdam -- the layer classes of BinaryBrain's LUT path, host side in C++, device side through
// the bbcu_* C ABI of libbbcu_b200.  Class names, create_t fields, command strings and defaults follow the
// reference (include/bb/DifferentiableLutN.h:86-162, StochasticLutN.h:36-121, BinaryLutN.h:30-140,
// StochasticBatchNormalization.h:67-137, OptimizerAdam.h:47-184).  There is no host_only/CPU branch: the
// "host_only" command is accepted and rejected with an error, because this build's operators are GPU-only.
#pragma once

#include <algorithm>
#include <cmath>
#include <deque>
#include <functional>
#include <random>
#include <string>

#include "Memory.h"
#include "Serialize.h"

namespace bb {

// ---------------------------------------------------------------------------------------------------
// Seeded wiring.  Same procedure as the reference's "random" rule (include/bb/ConnectionTable.h:268-280 with
// include/bb/ShuffleSet.h:27-103): deal N inputs per node from a shuffled deck of all input indices; when the
// deck runs out, reshuffle the already-dealt cards (those of the node being dealt last).  With libstdc++'s
// std::mt19937_64 / std::shuffle this reproduces the reference's tables for the same seed.
// ---------------------------------------------------------------------------------------------------
class ShuffleDeck
{
    std::mt19937_64     m_mt;
    std::deque<index_t> m_deck, m_used;

    void refill(std::vector<index_t> &from)
    {
        std::shuffle(from.begin(), from.end(), m_mt);
        m_deck.assign(from.begin(), from.end());
        from.clear();
    }

public:
    ShuffleDeck(index_t size, std::uint64_t seed) : m_mt(seed)
    {
        std::vector<index_t> all((std::size_t)size);
        for (std::size_t i = 0; i < all.size(); ++i) all[i] = (index_t)i;
        refill(all);
    }

    std::vector<index_t> Deal(index_t n)
    {
        std::vector<index_t> hand, stash;
        for (index_t i = 0; i < n; ++i) {
            if (m_deck.empty()) { std::vector<index_t> u(m_used.begin(), m_used.end()); m_used.clear(); refill(u); }
            if (m_deck.empty()) { refill(stash); }
            index_t card = m_deck.front();
            m_deck.pop_front();
            hand.push_back(card);
            stash.push_back(card);
        }
        for (auto c : stash) m_used.push_back(c);
        return hand;
    }
};

template <int N>
class FixedSizeConnectionTable
{
    index_t               m_in = 0, m_out = 0;
    Tensor_<std::int32_t> m_table;       // [out][N]

public:
    void SetShape(index_t in_nodes, index_t out_nodes) { m_in = in_nodes; m_out = out_nodes; m_table.Resize({out_nodes, N}); m_table.FillZero(); }
    index_t GetInputNodeSize()  const { return m_in; }
    index_t GetOutputNodeSize() const { return m_out; }

    // The reference's wiring rules (include/bb/ConnectionTable.h:150-284), selected by the first word of `rule`:
    //   "" / "random"  N distinct inputs per node dealt from one deck over all inputs;
    //   "serial"       inputs 0, 1, 2, ... in order, wrapping around;
    //   "pointwise"    shapes {c, h, w} with equal h, w: a node at (c, y, x) reads N channels of the same pixel (one deck per pixel);
    //   "depthwise"    equal channel counts: a node of channel c reads N pixels of channel c (one deck per channel);
    //   "gauss"        inputs drawn around the node's own (scaled) position with a normal distribution per axis, no repeats.
    // Node index of a position: row-major over the shape, last axis fastest.  The per-pixel / per-channel decks are seeded
    // from std::mt19937_64(seed) in visiting order, so libstdc++ builds give the reference's tables for the same seed.
    void InitializeConnection(std::uint64_t seed, std::string const &rule, indices_t const &in_shape, indices_t const &out_shape)
    {
        BB_ASSERT(CalcShapeSize(in_shape) == m_in && CalcShapeSize(out_shape) == m_out);
        auto t = m_table.Host(true);
        const std::string kind = rule.substr(0, rule.find(' '));
        auto flat = [](indices_t const &pos, indices_t const &shape) {
            index_t k = 0;
            for (std::size_t a = 0; a < shape.size(); ++a) k = k * shape[a] + pos[a];
            return k;
        };
        if (kind == "serial") {                                   // ConnectionTable.h:255-266
            index_t k = 0;
            for (index_t o = 0; o < m_out; ++o) for (int i = 0; i < N; ++i) t[o * N + i] = (std::int32_t)(k++ % m_in);
            return;
        }
        if (kind == "pointwise") {                                // ConnectionTable.h:160-181
            BB_ASSERT(in_shape.size() == 3 && out_shape.size() == 3 && in_shape[1] == out_shape[1] && in_shape[2] == out_shape[2]);
            std::mt19937_64 mt(seed);
            for (index_t y = 0; y < out_shape[1]; ++y)
                for (index_t x = 0; x < out_shape[2]; ++x) {
                    ShuffleDeck deck(in_shape[0], mt());
                    for (index_t c = 0; c < out_shape[0]; ++c) {
                        auto hand = deck.Deal(N);
                        const index_t o = flat({c, y, x}, out_shape);
                        for (int i = 0; i < N; ++i) t[o * N + i] = (std::int32_t)flat({hand[i], y, x}, in_shape);
                    }
                }
            return;
        }
        if (kind == "depthwise") {                                // ConnectionTable.h:183-210
            BB_ASSERT(in_shape.size() == 3 && out_shape.size() == 3 && in_shape[0] == out_shape[0]);
            std::mt19937_64 mt(seed);
            for (index_t c = 0; c < out_shape[0]; ++c) {
                ShuffleDeck deck(in_shape[1] * in_shape[2], mt());
                for (index_t y = 0; y < out_shape[1]; ++y)
                    for (index_t x = 0; x < out_shape[2]; ++x) {
                        auto hand = deck.Deal(N);
                        const index_t o = flat({c, y, x}, out_shape);
                        for (int i = 0; i < N; ++i) t[o * N + i] = (std::int32_t)flat({c, hand[i] / in_shape[2], hand[i] % in_shape[2]}, in_shape);
                    }
            }
            return;
        }
        if (kind == "gauss") {                                    // ConnectionTable.h:212-253
            const int n = (int)in_shape.size();
            BB_ASSERT((int)out_shape.size() == n);
            std::vector<double> step(n), sigma(n);
            for (int a = 0; a < n; ++a) {
                step[a]  = (double)(in_shape[a] - 1) / (double)(out_shape[a] - 1);      // 0/0 for an axis of one node on both sides, as in the reference
                sigma[a] = (double)in_shape[a] / (double)out_shape[a];
            }
            std::mt19937_64 mt(seed);
            std::normal_distribution<double> norm(0.0, 1.0);
            indices_t pos((std::size_t)n, 0);
            for (index_t o = 0; o < m_out; ++o) {                 // row-major visiting order = the node index
                std::vector<index_t> taken;
                for (int i = 0; i < N; ++i) {
                    for (;;) {
                        indices_t src((std::size_t)n);
                        for (int a = 0; a < n; ++a) {
                            double p = (double)pos[a] * step[a] + norm(mt) * sigma[a];
                            while (p < 0) p += (double)in_shape[a];                     // wrap negative positions, then truncate and wrap
                            src[a] = (index_t)p % in_shape[a];
                        }
                        const index_t in_node = flat(src, in_shape);
                        if (std::find(taken.begin(), taken.end(), in_node) == taken.end()) {
                            t[o * N + i] = (std::int32_t)in_node;
                            taken.push_back(in_node);
                            break;
                        }
                    }
                }
                for (int a = n - 1; a >= 0; --a) { if (++pos[a] < out_shape[a]) break; pos[a] = 0; }
            }
            return;
        }
        if (!(kind.empty() || kind == "random")) throw std::runtime_error("unknown connection rule : \"" + kind + "\"");
        ShuffleDeck deck(m_in, seed);                             // ConnectionTable.h:268-280
        for (index_t o = 0; o < m_out; ++o) {
            auto hand = deck.Deal(N);
            for (int i = 0; i < N; ++i) t[o * N + i] = (std::int32_t)hand[i];
        }
    }
    void InitializeConnection(std::uint64_t seed, std::string const &rule = "") { InitializeConnection(seed, rule, indices_t({m_in}), indices_t({m_out})); }
    index_t GetInputConnection(index_t node, int i) const { return m_table.HostConst()[node * N + i]; }
    void    SetInputConnection(index_t node, int i, index_t in_node)
    {
        BB_ASSERT(in_node >= 0 && in_node < m_in && node >= 0 && node < m_out && i >= 0 && i < N);
        m_table.Host()[node * N + i] = (std::int32_t)in_node;
    }
    std::int32_t const *LockDeviceMemConst_InputTable() const { return m_table.DevConst(); }
    Tensor_<std::int32_t> &Table() { return m_table; }

    // include/bb/FixedSizeConnectionTable.h:50-61 over include/bb/ConnectionTable.h (shapes) over Object
    void DumpObject(std::ostream &os, indices_t const &in_shape, indices_t const &out_shape) const
    {
        serial::WriteHeader(os, "FixedSizeConnectionTable" + std::to_string(N) + "_int32");
        serial::Save(os, (std::int64_t)1);
        serial::Save(os, (std::int64_t)1);
        serial::Save(os, (std::int64_t)0);
        serial::SaveShape(os, in_shape);
        serial::SaveShape(os, out_shape);
        serial::DumpTypedTensor(os, m_table);
    }
    void LoadObject(std::istream &is)
    {
        serial::ReadHeader(is, "FixedSizeConnectionTable" + std::to_string(N) + "_int32");
        serial::ExpectVersion(is, 1, "FixedSizeConnectionTable");
        serial::ExpectVersion(is, 1, "ConnectionTable");
        serial::ExpectVersion(is, 0, "Object");
        indices_t in_shape = serial::LoadShape(is), out_shape = serial::LoadShape(is);
        m_in = CalcShapeSize(in_shape); m_out = CalcShapeSize(out_shape);
        serial::LoadTypedTensor(is, m_table);
        if (m_table.GetShape() != indices_t({m_out, (index_t)N})) throw std::runtime_error("LoadObject: connection table shape");
        std::int32_t const *t = m_table.HostConst();
        for (index_t i = 0; i < m_out * N; ++i)
            if (t[i] < 0 || t[i] >= m_in) throw std::runtime_error("LoadObject: connection index out of range");
    }
};


// ---------------------------------------------------------------------------------------------------
// Model base: command strings and the saved-input stack (include/bb/Model.h:62-120,400-440)
// ---------------------------------------------------------------------------------------------------
class Model
{
protected:
    std::vector<FrameBuffer> m_stack;
    bool m_parameter_lock = false;
    std::string m_name;

    static bool EvalBool(std::string const &s) { return s == "true" || s == "True" || s == "TRUE" || s == "1"; }
    virtual void CommandProc(std::vector<std::string> const &args)
    {
        if (args.size() == 2 && args[0] == "parameter_lock") m_parameter_lock = EvalBool(args[1]);
        if (args.size() == 2 && args[0] == "host_only" && EvalBool(args[1]))
            throw std::runtime_error("host_only true: this build has no CPU branch behind the bbcu_* operators");
    }

public:
    virtual ~Model() {}
    virtual std::string GetModelName() const = 0;
    virtual std::string GetObjectName() const { return GetModelName(); }
    void SetName(std::string const &name) { m_name = name; }
    std::string GetName() const { return m_name.empty() ? GetModelName() : m_name; }

    // Serialisation in the reference's object format (include/bb/Object.h:38-58): layers dumped by BinaryBrain load here and back.
    virtual void DumpObjectData(std::ostream &) const { throw std::runtime_error(GetModelName() + ": DumpObject is not provided"); }
    virtual void LoadObjectData(std::istream &)       { throw std::runtime_error(GetModelName() + ": LoadObject is not provided"); }
    void DumpObject(std::ostream &os) const { serial::WriteHeader(os, GetObjectName()); DumpObjectData(os); }
    void LoadObject(std::istream &is)       { serial::ReadHeader(is, GetObjectName()); LoadObjectData(is); }
    std::string DumpObjectBytes() const { std::ostringstream os(std::ios::binary); DumpObject(os); return os.str(); }
    void LoadObjectBytes(std::string const &bytes) { std::istringstream is(bytes, std::ios::binary); LoadObject(is); }
    virtual indices_t SetInputShape(indices_t shape) = 0;
    virtual indices_t GetInputShape() const = 0;
    virtual indices_t GetOutputShape() const = 0;
    virtual FrameBuffer Forward(FrameBuffer x, bool train = true) = 0;
    virtual FrameBuffer Backward(FrameBuffer dy) = 0;
    index_t GetInputNodeSize()  const { return CalcShapeSize(GetInputShape()); }
    index_t GetOutputNodeSize() const { return CalcShapeSize(GetOutputShape()); }

    void SendCommand(std::string const &command)
    {
        std::vector<std::string> args;
        std::istringstream is(command);
        for (std::string a; is >> a;) args.push_back(a);
        CommandProc(args);
    }
    void PushFrameBuffer(FrameBuffer b) { m_stack.push_back(b); }
    FrameBuffer PopFrameBuffer() { BB_ASSERT(!m_stack.empty()); FrameBuffer b = m_stack.back(); m_stack.pop_back(); return b; }
    virtual void Clear() { m_stack.clear(); }
};


// Shared state of the two differentiable LUT layers: wiring, W, dW.
template <int N>
class SparseLutBase : public Model
{
protected:
    static constexpr int NN = 1 << N;
    indices_t                   m_input_shape, m_output_shape;
    FixedSizeConnectionTable<N> m_connection_table;
    std::string                 m_connection;
    std::shared_ptr<Tensor>     m_W = std::make_shared<Tensor>(), m_dW = std::make_shared<Tensor>();
    std::mt19937_64             m_mt;
    float                       m_unbinarize_bias = 0.25f;
    bool                        m_lut_binarize = false;
    bool                        m_binary_mode  = true;

    void init_parameters(indices_t shape)
    {
        m_input_shape = shape;
        m_connection_table.SetShape(CalcShapeSize(m_input_shape), CalcShapeSize(m_output_shape));
        m_connection_table.InitializeConnection(m_mt(), m_connection, m_input_shape, m_output_shape);
        // W ~ N(0.5, 0.01) drawn in double and narrowed (include/bb/Tensor.h:555-565, DifferentiableLutN.h:495)
        m_W->Resize({CalcShapeSize(m_output_shape), NN});
        {
            std::mt19937_64 mt(m_mt());
            std::normal_distribution<double> dist(0.5, 0.01);
            float *w = m_W->Host(true);
            for (index_t i = 0; i < m_W->GetSize(); ++i) w[i] = (float)dist(mt);
        }
        m_dW->Resize({CalcShapeSize(m_output_shape), NN});
        m_dW->FillZero();
    }

public:
    indices_t GetInputShape()  const override { return m_input_shape; }
    indices_t GetOutputShape() const override { return m_output_shape; }
    Tensor &W()  { return *m_W; }
    Tensor &dW() { return *m_dW; }
    std::shared_ptr<Tensor> GetParameters() { return m_W; }
    std::shared_ptr<Tensor> GetGradients()  { return m_dW; }
    index_t GetNodeConnectionSize(index_t) const { return N; }
    index_t GetNodeConnectionIndex(index_t node, index_t i) const { return m_connection_table.GetInputConnection(node, (int)i); }
    void    SetNodeConnectionIndex(index_t node, index_t i, index_t in_node) { m_connection_table.SetInputConnection(node, (int)i, in_node); }
    FixedSizeConnectionTable<N> &ConnectionTable() { return m_connection_table; }
};


// ---------------------------------------------------------------------------------------------------
// DifferentiableLutN<6, BinType, float>: LUT6 + fused batch norm (+ binarize / hard-tanh)
// ---------------------------------------------------------------------------------------------------
template <int N = 6, typename BinType = float, typename RealType = float>
class DifferentiableLutN : public SparseLutBase<N>
{
    static_assert(N == 6, "libbbcu_b200 implements the 6-input LUT");
    using _super = SparseLutBase<N>;
    static constexpr bool kBit = std::is_same<BinType, Bit>::value;

    bool  m_batch_norm = true, m_backward_break = false, m_flagClamp = false;
    float m_momentum, m_gamma, m_beta;
    Tensor m_mean, m_rstd, m_running_mean, m_running_var;

public:
    // Adds, over all ranks, `count` doubles / floats that live in DEVICE memory, in place and in order on `stream` (with NCCL:
    // ncclAllReduce(p, p, count, ncclDouble / ncclFloat, ncclSum, comm, stream)).  Injected so that this header needs no
    // communication library.
    using AllReduceF64 = std::function<void(double *dev, std::size_t count, cudaStream_t stream)>;
    using AllReduceF32 = std::function<void(float *dev, std::size_t count, cudaStream_t stream)>;

private:
    index_t        m_total_frames = 0;          // > 0: this object holds one frame shard of a batch of that many frames
    AllReduceF64   m_allreduce_sums;
    AllReduceF32   m_allreduce_grads;
    Tensor_<double> m_sums;                     // [O][2] batch sums on their way through the exchange
    std::vector<FrameBuffer> m_y_stack;         // training outputs, kept for the backward statistics (probability mode); pushed and
                                                // popped with the inputs, so several forwards may precede their backwards

public:
    struct create_t {
        indices_t     output_shape;
        bool          batch_norm = true;
        bool          binary     = true;
        std::string   connection;
        float         momentum   = 0.9f;
        float         gamma      = 0.3f;
        float         beta       = 0.5f;
        std::uint64_t seed       = 1;
    };

    explicit DifferentiableLutN(create_t const &c)
    {
        this->m_output_shape = c.output_shape;
        this->m_connection   = c.connection;
        this->m_binary_mode  = kBit ? true : c.binary;
        this->m_mt.seed(c.seed);
        m_batch_norm = c.batch_norm;
        m_momentum = c.momentum; m_gamma = c.gamma; m_beta = c.beta;
    }
    static std::shared_ptr<DifferentiableLutN> Create(create_t const &c) { return std::make_shared<DifferentiableLutN>(c); }
    static std::shared_ptr<DifferentiableLutN> Create(index_t out, bool batch_norm = true, std::string connection = "")
    {
        create_t c; c.output_shape = {out}; c.batch_norm = batch_norm; c.connection = connection;
        return Create(c);
    }
    // Python-side defaults differ from the C++ ones: momentum 0.0 (include/bb/DifferentiableLutN.h:208-228)
    static std::shared_ptr<DifferentiableLutN> CreatePy(indices_t output_shape, bool batch_norm = true, bool binary = true,
                                                        std::string connection = "", double momentum = 0.0, double gamma = 0.3,
                                                        double beta = 0.5, std::uint64_t seed = 1)
    {
        create_t c; c.output_shape = output_shape; c.batch_norm = batch_norm; c.binary = binary; c.connection = connection;
        c.momentum = (float)momentum; c.gamma = (float)gamma; c.beta = (float)beta; c.seed = seed;
        return Create(c);
    }

    // Frame sharding (no counterpart in the reference, which has no multi-device path: include/bb/Memory.h:215-216).  After this
    // call Forward(train) / Backward treat their buffers as ONE SHARD of a batch of total_frames frames that is spread over the
    // ranks of a job: the batch-norm statistics of both passes are formed from per-rank sums that `allreduce_sums` adds over
    // the ranks ([output nodes][2] fp64, twice per step, on the critical path), and, when `allreduce_grads` is given, the
    // table gradients are added over the ranks at the end of Backward.  fp32 frames with batch norm only.  total_frames = 0
    // switches sharding off again.
    void SetFrameShard(index_t total_frames, AllReduceF64 allreduce_sums, AllReduceF32 allreduce_grads = nullptr)
    {
        BB_ASSERT(!kBit && m_batch_norm);
        BB_ASSERT(total_frames == 0 || static_cast<bool>(allreduce_sums));
        m_total_frames = total_frames;
        m_allreduce_sums = allreduce_sums;
        m_allreduce_grads = allreduce_grads;
    }
    index_t GetTotalFrames() const { return m_total_frames; }

    std::string GetModelName() const override { return "DifferentiableLut" + std::to_string(N); }
    std::string GetObjectName() const override { return GetModelName() + "_" + DataType<BinType>::Name() + "_" + DataType<RealType>::Name(); }

    Tensor &running_mean() { return m_running_mean; }
    Tensor &running_var()  { return m_running_var; }
    Tensor &tmp_mean()     { return m_mean; }
    Tensor &tmp_rstd()     { return m_rstd; }
    float GetGamma() const { return m_gamma; }
    float GetBeta()  const { return m_beta; }

    // One node on the host, with the running statistics (include/bb/DifferentiableLutN.h:527-586): the value a frozen node takes for
    // six given inputs -- what the reference uses when it exports a trained network to a truth table.  Same product form as
    // StochasticOperation_Lut_Forward (include/bb/StochasticOperation.h:95-114).
    std::vector<double> ForwardNode(index_t node, std::vector<double> input_value) const
    {
        BB_ASSERT((int)input_value.size() == N && node >= 0 && node < CalcShapeSize(this->m_output_shape));
        float const *Wp = this->m_W->HostConst() + node * _super::NN;
        float x[N];
        for (int i = 0; i < N; ++i) {
            x[i] = (float)input_value[i];
            if (this->m_binary_mode) x[i] = 0.5f + ((x[i] > 0.5f) ? +this->m_unbinarize_bias : -this->m_unbinarize_bias);
            else                     x[i] = std::min(1.0f, std::max(0.0f, x[i]));
        }
        float y = 0.0f;
        for (int i = 0; i < _super::NN; ++i) {
            float w = std::min(1.0f, std::max(0.0f, Wp[i]));                      // the clamp Forward applies to the parameters
            if (this->m_lut_binarize) w = w > 0.5f ? 1.0f : 0.0f;
            for (int j = 0; j < N; ++j) w *= ((i >> j) & 1) ? x[j] : (1.0f - x[j]);
            y += w;
        }
        if (m_batch_norm) {
            float rstd = 1.0f / std::sqrt(m_running_var.HostConst()[node]);
            y = (y - m_running_mean.HostConst()[node]) * rstd;
            y = y * m_gamma + m_beta;
        }
        if (this->m_binary_mode) y = y > 0.5f ? 1.0f : 0.0f;
        else                     y = std::max(std::min(y, 1.0f), 0.0f);
        return std::vector<double>{(double)y};
    }

    // include/bb/DifferentiableLutN.h:264-330
    void DumpObjectData(std::ostream &os) const override
    {
        serial::Save(os, (std::int64_t)1);
        serial::SaveModelBase(os, this->m_name);
        serial::SaveBool(os, false);                         // host_only: there is no host branch here
        serial::SaveBool(os, this->m_lut_binarize);
        serial::SaveBool(os, this->m_binary_mode);
        serial::SaveBool(os, m_batch_norm);
        serial::SaveBool(os, m_flagClamp);
        serial::SaveShape(os, this->m_input_shape);
        serial::SaveShape(os, this->m_output_shape);
        this->m_connection_table.DumpObject(os, this->m_input_shape, this->m_output_shape);
        serial::DumpTensor(os, *this->m_W);
        serial::Save(os, this->m_unbinarize_bias);
        serial::Save(os, m_momentum);
        serial::Save(os, m_gamma);
        serial::Save(os, m_beta);
        serial::DumpTypedTensor(os, m_running_mean);
        serial::DumpTypedTensor(os, m_running_var);
    }
    void LoadObjectData(std::istream &is) override
    {
        serial::ExpectVersion(is, 1, "DifferentiableLutN");
        this->m_name = serial::LoadModelBase(is);
        (void)serial::LoadBool(is);                          // host_only
        this->m_lut_binarize = serial::LoadBool(is);
        this->m_binary_mode  = serial::LoadBool(is) || kBit;
        m_batch_norm = serial::LoadBool(is);
        m_flagClamp  = serial::LoadBool(is);
        this->m_input_shape  = serial::LoadShape(is);
        this->m_output_shape = serial::LoadShape(is);
        this->m_connection_table.LoadObject(is);
        serial::LoadTensor(is, *this->m_W);
        serial::Load(is, this->m_unbinarize_bias);
        serial::Load(is, m_momentum);
        serial::Load(is, m_gamma);
        serial::Load(is, m_beta);
        serial::LoadTypedTensor(is, m_running_mean);
        serial::LoadTypedTensor(is, m_running_var);
        index_t O = CalcShapeSize(this->m_output_shape);
        if (this->m_W->GetShape() != indices_t({O, (index_t)_super::NN}) || m_running_mean.GetSize() != O || m_running_var.GetSize() != O ||
            this->m_connection_table.GetOutputNodeSize() != O || this->m_connection_table.GetInputNodeSize() != CalcShapeSize(this->m_input_shape))
            throw std::runtime_error("LoadObject: inconsistent layer shapes");
        this->m_dW->Resize(this->m_W->GetShape());
        this->m_dW->FillZero();
        m_mean.Resize(O); m_rstd.Resize(O);
    }

    indices_t SetInputShape(indices_t shape) override
    {
        if (shape == this->m_input_shape) return this->m_output_shape;
        this->init_parameters(shape);
        index_t O = CalcShapeSize(this->m_output_shape);
        m_mean.Resize(O); m_rstd.Resize(O);
        m_running_mean.Resize(O); m_running_mean.Fill(0.0f);
        m_running_var.Resize(O);  m_running_var.Fill(1.0f);
        return this->m_output_shape;
    }

    FrameBuffer Forward(FrameBuffer x_buf, bool train = true) override
    {
        if (x_buf.GetShape() != this->m_input_shape) SetInputShape(x_buf.GetShape());
        BB_ASSERT(x_buf.GetType() == DataType<BinType>::type);
        FrameBuffer y_buf(x_buf.GetFrameSize(), this->m_output_shape, DataType<BinType>::type);
        if (train) this->PushFrameBuffer(x_buf);
        cudaStream_t st = Manager::Stream();
        if (m_flagClamp) {        // DifferentiableLutN.h:605-608
            BBCU_CHECK(bbcu_fp32_Vector_clamp(this->m_W->Dev(), this->m_W->DevConst(), 0.0f, 1.0f, (int)this->m_W->GetSize(), st));
            m_flagClamp = false;
        }
        int O = (int)y_buf.GetNodeSize(), F = (int)y_buf.GetFrameSize();
        int ys = (int)(y_buf.GetFrameStride() / 4), xs = (int)(x_buf.GetFrameStride() / 4);
        auto idx = this->m_connection_table.LockDeviceMemConst_InputTable();
        if (m_batch_norm) {
            if (kBit) {
                BB_ASSERT(xs == ys);
                if (train) BBCU_CHECK(bbcu_bit_fp32_DifferentiableLut6_ForwardTraining(
                        (int const *)x_buf.LockDeviceMemoryConst(), (int *)y_buf.LockDeviceMemory(true), idx, this->m_W->DevConst(), m_mean.Dev(true),
                        m_rstd.Dev(true), m_running_mean.Dev(), m_running_var.Dev(), m_gamma, m_beta, m_momentum, this->m_unbinarize_bias, O, F, ys,
                        this->m_lut_binarize, st));
                else BBCU_CHECK(bbcu_bit_fp32_DifferentiableLut6_ForwardInference(
                        (int const *)x_buf.LockDeviceMemoryConst(), (int *)y_buf.LockDeviceMemory(true), idx, this->m_W->DevConst(),
                        m_running_mean.DevConst(), m_running_var.DevConst(), m_gamma, m_beta, this->m_unbinarize_bias, O, F, ys, this->m_lut_binarize, st));
            } else if (train && m_total_frames > 0) {
                // one shard of a larger batch: raw values and per-rank sums, the exchange, then the normalisation with the batch statistics
                BB_ASSERT(xs == ys && m_total_frames >= F);
                m_sums.Resize({(index_t)O, 2});
                BBCU_CHECK(bbcu_fp32_DifferentiableLut6_ForwardStats(
                        (float const *)x_buf.LockDeviceMemoryConst(), (float *)y_buf.LockDeviceMemory(true), idx, this->m_W->DevConst(), m_sums.Dev(true),
                        this->m_unbinarize_bias, O, F, ys, this->m_lut_binarize, this->m_binary_mode, st));
                m_allreduce_sums(m_sums.Dev(), (std::size_t)O * 2, st);
                BBCU_CHECK(bbcu_fp32_DifferentiableLut6_ForwardNormalize(
                        (float *)y_buf.LockDeviceMemory(), m_sums.DevConst(), m_mean.Dev(true), m_rstd.Dev(true), m_running_mean.Dev(), m_running_var.Dev(),
                        m_gamma, m_beta, m_momentum, O, F, ys, (long long)m_total_frames, this->m_binary_mode, st));
                m_y_stack.push_back(this->m_binary_mode ? FrameBuffer() : y_buf);
            } else {
                BB_ASSERT(xs == ys);
                if (train) {
                    BBCU_CHECK(bbcu_fp32_DifferentiableLut6_ForwardTraining(
                        (float const *)x_buf.LockDeviceMemoryConst(), (float *)y_buf.LockDeviceMemory(true), idx, this->m_W->DevConst(), m_mean.Dev(true),
                        m_rstd.Dev(true), m_running_mean.Dev(), m_running_var.Dev(), m_gamma, m_beta, m_momentum, this->m_unbinarize_bias, O, F, ys,
                        this->m_lut_binarize, this->m_binary_mode, st));
                    // probability mode: the backward takes its batch-norm sums from this output (8 bytes per node-frame) instead of
                    // evaluating the LUT a second time; the buffer is the one the next layer holds anyway
                    m_y_stack.push_back(this->m_binary_mode ? FrameBuffer() : y_buf);
                }
                else BBCU_CHECK(bbcu_fp32_DifferentiableLut6_ForwardInference(
                        (float const *)x_buf.LockDeviceMemoryConst(), (float *)y_buf.LockDeviceMemory(true), idx, this->m_W->DevConst(),
                        m_running_mean.DevConst(), m_running_var.DevConst(), m_gamma, m_beta, this->m_unbinarize_bias, O, F, ys, this->m_lut_binarize,
                        this->m_binary_mode, st));
            }
        } else {
            // batch_norm=false: the plain stochastic LUT (DifferentiableLutN.h:907-1010)
            if (kBit) BBCU_CHECK(bbcu_bit_bit_fp32_StochasticLut6_Forward((int const *)x_buf.LockDeviceMemoryConst(), (int *)y_buf.LockDeviceMemory(true),
                                                                          idx, this->m_W->DevConst(), O, F, ys, this->m_lut_binarize,
                                                                          this->m_unbinarize_bias, st));
            else      BBCU_CHECK(bbcu_fp32_StochasticLut6_Forward((float const *)x_buf.LockDeviceMemoryConst(), (float *)y_buf.LockDeviceMemory(true), idx,
                                                                  this->m_W->DevConst(), O, F, ys, this->m_binary_mode, this->m_lut_binarize,
                                                                  this->m_unbinarize_bias, st));
        }
        return y_buf;
    }

    FrameBuffer Backward(FrameBuffer dy_buf) override
    {
        if (m_backward_break || dy_buf.Empty()) { this->m_dW->FillZero(); return FrameBuffer(); }
        BB_ASSERT(dy_buf.GetType() == BB_TYPE_FP32);
        m_flagClamp = true;
        FrameBuffer x_buf = this->PopFrameBuffer();
        FrameBuffer dx_buf(dy_buf.GetFrameSize(), this->m_input_shape, BB_TYPE_FP32);
        cudaStream_t st = Manager::Stream();
        int I = (int)dx_buf.GetNodeSize(), O = (int)dy_buf.GetNodeSize(), F = (int)dy_buf.GetFrameSize();
        int fs = (int)(dy_buf.GetFrameStride() / 4), xs = (int)(x_buf.GetFrameStride() / 4);
        auto idx = this->m_connection_table.LockDeviceMemConst_InputTable();
        FrameBuffer y_saved;
        if (!m_y_stack.empty()) { y_saved = m_y_stack.back(); m_y_stack.pop_back(); }
        const bool from_output = !this->m_binary_mode && !y_saved.Empty() && y_saved.GetFrameSize() == dy_buf.GetFrameSize();
        if (m_batch_norm && !kBit && (m_total_frames > 0 || from_output)) {
            // the two halves of the backward: per-rank sums, their exchange when this object holds a frame shard, then the gradients
            const long long total = m_total_frames > 0 ? (long long)m_total_frames : (long long)F;
            Tensor dmean(indices_t{O}), dvar(indices_t{O});
            m_sums.Resize({(index_t)O, 2});
            float const *xp = (float const *)x_buf.LockDeviceMemoryConst(), *dyp = (float const *)dy_buf.LockDeviceMemoryConst();
            if (from_output) {
                // probability mode: the sums come from the saved output (8 bytes per node-frame) instead of a second LUT evaluation
                BBCU_CHECK(bbcu_fp32_DifferentiableLut6_BackwardStatsFromOutput((float const *)y_saved.LockDeviceMemoryConst(), dyp, m_rstd.DevConst(),
                                                                                m_sums.Dev(true), m_gamma, m_beta, O, F, fs, 0, st));
            } else {
                BBCU_CHECK(bbcu_fp32_DifferentiableLut6_BackwardStats(xp, dyp, idx, this->m_W->DevConst(), m_mean.DevConst(), m_rstd.DevConst(),
                                                                      m_sums.Dev(true), m_gamma, m_beta, this->m_unbinarize_bias, O, F, fs,
                                                                      this->m_lut_binarize, this->m_binary_mode, st));
            }
            y_saved = FrameBuffer();
            if (m_total_frames > 0) m_allreduce_sums(m_sums.Dev(), (std::size_t)O * 2, st);
            BBCU_CHECK(bbcu_fp32_DifferentiableLut6_BackwardApply(xp, dyp, (float *)dx_buf.LockDeviceMemory(true), idx, this->m_W->DevConst(),
                                                                  this->m_dW->Dev(), m_mean.DevConst(), m_rstd.DevConst(), m_sums.DevConst(),
                                                                  dmean.Dev(true), dvar.Dev(true), m_gamma, m_beta, this->m_unbinarize_bias, I, O, F, fs,
                                                                  total, this->m_lut_binarize, this->m_binary_mode, st));
            if (m_total_frames > 0 && m_allreduce_grads) m_allreduce_grads(this->m_dW->Dev(), (std::size_t)this->m_dW->GetSize(), st);
        } else if (m_batch_norm) {
            Tensor dmean(indices_t{O}), dvar(indices_t{O});
            if (kBit) BBCU_CHECK(bbcu_bit_fp32_DifferentiableLut6_Backward(
                    (int const *)x_buf.LockDeviceMemoryConst(), (float const *)dy_buf.LockDeviceMemoryConst(), (float *)dx_buf.LockDeviceMemory(true), nullptr,
                    idx, nullptr, this->m_W->DevConst(), this->m_dW->Dev(), m_mean.DevConst(), m_rstd.DevConst(), dmean.Dev(true), dvar.Dev(true),
                    m_gamma, m_beta, this->m_unbinarize_bias, 0, I, O, F, fs, xs, 0, 0, this->m_lut_binarize, st));
            else      BBCU_CHECK(bbcu_fp32_DifferentiableLut6_Backward(
                    (float const *)x_buf.LockDeviceMemoryConst(), (float const *)dy_buf.LockDeviceMemoryConst(), (float *)dx_buf.LockDeviceMemory(true), nullptr,
                    idx, nullptr, this->m_W->DevConst(), this->m_dW->Dev(), m_mean.DevConst(), m_rstd.DevConst(), dmean.Dev(true), dvar.Dev(true),
                    m_gamma, m_beta, this->m_unbinarize_bias, 0, I, O, F, fs, 0, 0, this->m_lut_binarize, this->m_binary_mode, st));
            // dmean / dvar return to the heap cache here; the heap never cudaFree()s behind running work, and a later owner of
            // the block enqueues on the same layer stream, i.e. after the kernels above
        } else {
            if (kBit) BBCU_CHECK(bbcu_bit_fp32_StochasticLut6_Backward(
                    (int const *)x_buf.LockDeviceMemoryConst(), (float const *)dy_buf.LockDeviceMemoryConst(), (float *)dx_buf.LockDeviceMemory(true), nullptr,
                    idx, nullptr, this->m_W->DevConst(), this->m_dW->Dev(), 0, I, O, F, fs, xs, 0, 0, this->m_lut_binarize, this->m_unbinarize_bias, st));
            else      BBCU_CHECK(bbcu_fp32_StochasticLut6_Backward(
                    (float const *)x_buf.LockDeviceMemoryConst(), (float const *)dy_buf.LockDeviceMemoryConst(), (float *)dx_buf.LockDeviceMemory(true), nullptr,
                    idx, nullptr, this->m_W->DevConst(), this->m_dW->Dev(), 0, I, O, F, fs, 0, 0, this->m_binary_mode, this->m_lut_binarize,
                    this->m_unbinarize_bias, st));
        }
        return dx_buf;
    }

    void Clear() override { Model::Clear(); m_y_stack.clear(); }

protected:
    void CommandProc(std::vector<std::string> const &args) override
    {
        Model::CommandProc(args);
        if (args.size() != 2) return;
        if (!kBit && args[0] == "binary")   this->m_binary_mode = Model::EvalBool(args[1]);
        if (args[0] == "lut_binarize")      this->m_lut_binarize = Model::EvalBool(args[1]);
        if (args[0] == "batch_norm")        m_batch_norm = Model::EvalBool(args[1]);
        if (args[0] == "momentum")          m_momentum = std::stof(args[1]);
        if (args[0] == "backward_break")    m_backward_break = Model::EvalBool(args[1]);
    }
};


// ---------------------------------------------------------------------------------------------------
// StochasticLutN<6, BinType, float>: LUT6 without batch norm; fp32 output; W clamped every forward
// ---------------------------------------------------------------------------------------------------
template <int N = 6, typename BinType = float, typename RealType = float>
class StochasticLutN : public SparseLutBase<N>
{
    static_assert(N == 6, "libbbcu_b200 implements the 6-input LUT");
    static constexpr bool kBit = std::is_same<BinType, Bit>::value;
    FrameBuffer m_x_buf;

public:
    struct create_t {
        indices_t     output_shape;
        std::string   connection;
        std::uint64_t seed = 1;
    };
    explicit StochasticLutN(create_t const &c)
    {
        this->m_output_shape = c.output_shape;
        this->m_connection   = c.connection;
        this->m_mt.seed(c.seed);
        this->m_binary_mode  = kBit;                 // StochasticLutN.h:44
        this->m_lut_binarize = true;                 // StochasticLutN.h:45
    }
    static std::shared_ptr<StochasticLutN> Create(create_t const &c) { return std::make_shared<StochasticLutN>(c); }
    static std::shared_ptr<StochasticLutN> Create(index_t out, std::string connection = "", std::uint64_t seed = 1)
    {
        create_t c; c.output_shape = {out}; c.connection = connection; c.seed = seed;
        return Create(c);
    }
    static std::shared_ptr<StochasticLutN> CreatePy(indices_t output_shape, std::string connection = "", std::uint64_t seed = 1)
    {
        create_t c; c.output_shape = output_shape; c.connection = connection; c.seed = seed;
        return Create(c);
    }
    std::string GetModelName() const override { return "StochasticLut" + std::to_string(N); }
    std::string GetObjectName() const override { return GetModelName() + "_" + DataType<BinType>::Name() + "_" + DataType<RealType>::Name(); }

    // include/bb/StochasticLutN.h:170-230
    void DumpObjectData(std::ostream &os) const override
    {
        serial::Save(os, (std::int64_t)1);
        serial::SaveModelBase(os, this->m_name);
        serial::SaveBool(os, false);                         // host_only
        serial::SaveBool(os, true);                          // host_simd (the reference's default; no host branch here)
        serial::SaveBool(os, this->m_binary_mode);
        serial::SaveBool(os, this->m_lut_binarize);
        serial::SaveBool(os, false);                         // y_binarize
        serial::Save(os, (std::int64_t)(256 * 1024 * 1024)); // max_tmp_mem_size (unused: no dx temporary)
        serial::SaveString(os, this->m_connection);
        serial::Save(os, this->m_unbinarize_bias);
        serial::SaveShape(os, this->m_input_shape);
        serial::SaveShape(os, this->m_output_shape);
        this->m_connection_table.DumpObject(os, this->m_input_shape, this->m_output_shape);
        serial::DumpTensor(os, *this->m_W);
    }
    void LoadObjectData(std::istream &is) override
    {
        serial::ExpectVersion(is, 1, "StochasticLutN");
        this->m_name = serial::LoadModelBase(is);
        (void)serial::LoadBool(is);
        (void)serial::LoadBool(is);
        this->m_binary_mode  = serial::LoadBool(is) || kBit;
        this->m_lut_binarize = serial::LoadBool(is);
        if (serial::LoadBool(is)) throw std::runtime_error("LoadObject: y_binarize layers are not provided");
        std::int64_t tmp; serial::Load(is, tmp);
        this->m_connection = serial::LoadString(is);
        serial::Load(is, this->m_unbinarize_bias);
        this->m_input_shape  = serial::LoadShape(is);
        this->m_output_shape = serial::LoadShape(is);
        this->m_connection_table.LoadObject(is);
        serial::LoadTensor(is, *this->m_W);
        index_t O = CalcShapeSize(this->m_output_shape);
        if (this->m_W->GetShape() != indices_t({O, (index_t)SparseLutBase<N>::NN}) || this->m_connection_table.GetOutputNodeSize() != O ||
            this->m_connection_table.GetInputNodeSize() != CalcShapeSize(this->m_input_shape))
            throw std::runtime_error("LoadObject: inconsistent layer shapes");
        this->m_dW->Resize(this->m_W->GetShape());
        this->m_dW->FillZero();
    }

    indices_t SetInputShape(indices_t shape) override
    {
        if (shape == this->m_input_shape) return this->m_output_shape;
        this->init_parameters(shape);
        return this->m_output_shape;
    }

    FrameBuffer Forward(FrameBuffer x_buf, bool train = true) override
    {
        BB_ASSERT(x_buf.GetType() == DataType<BinType>::type);
        if (x_buf.GetShape() != this->m_input_shape) SetInputShape(x_buf.GetShape());
        FrameBuffer y_buf(x_buf.GetFrameSize(), this->m_output_shape, BB_TYPE_FP32);
        if (train) m_x_buf = x_buf;
        cudaStream_t st = Manager::Stream();
        BBCU_CHECK(bbcu_fp32_Vector_clamp(this->m_W->Dev(), this->m_W->DevConst(), 0.0f, 1.0f, (int)this->m_W->GetSize(), st));   // StochasticLutN.h:451
        int O = (int)y_buf.GetNodeSize(), F = (int)y_buf.GetFrameSize(), ys = (int)(y_buf.GetFrameStride() / 4), xs = (int)(x_buf.GetFrameStride() / 4);
        auto idx = this->m_connection_table.LockDeviceMemConst_InputTable();
        if (kBit) BBCU_CHECK(bbcu_bit_fp32_StochasticLut6_Forward((int const *)x_buf.LockDeviceMemoryConst(), (float *)y_buf.LockDeviceMemory(true), idx,
                                                                  this->m_W->DevConst(), O, F, ys, xs, this->m_lut_binarize, this->m_unbinarize_bias, st));
        else      BBCU_CHECK(bbcu_fp32_StochasticLut6_Forward((float const *)x_buf.LockDeviceMemoryConst(), (float *)y_buf.LockDeviceMemory(true), idx,
                                                              this->m_W->DevConst(), O, F, ys, this->m_binary_mode, this->m_lut_binarize,
                                                              this->m_unbinarize_bias, st));
        return y_buf;
    }

    FrameBuffer Backward(FrameBuffer dy_buf) override
    {
        if (dy_buf.Empty()) { this->m_dW->FillZero(); return FrameBuffer(); }
        BB_ASSERT(dy_buf.GetType() == BB_TYPE_FP32);
        FrameBuffer x_buf = m_x_buf;
        m_x_buf = FrameBuffer();
        BB_ASSERT(!x_buf.Empty());
        FrameBuffer dx_buf(dy_buf.GetFrameSize(), this->m_input_shape, BB_TYPE_FP32);
        cudaStream_t st = Manager::Stream();
        int I = (int)dx_buf.GetNodeSize(), O = (int)dy_buf.GetNodeSize(), F = (int)dy_buf.GetFrameSize();
        int fs = (int)(dy_buf.GetFrameStride() / 4), xs = (int)(x_buf.GetFrameStride() / 4);
        auto idx = this->m_connection_table.LockDeviceMemConst_InputTable();
        if (kBit) BBCU_CHECK(bbcu_bit_fp32_StochasticLut6_Backward(
                (int const *)x_buf.LockDeviceMemoryConst(), (float const *)dy_buf.LockDeviceMemoryConst(), (float *)dx_buf.LockDeviceMemory(true), nullptr, idx,
                nullptr, this->m_W->DevConst(), this->m_dW->Dev(), 0, I, O, F, fs, xs, 0, 0, this->m_lut_binarize, this->m_unbinarize_bias, st));
        else      BBCU_CHECK(bbcu_fp32_StochasticLut6_Backward(
                (float const *)x_buf.LockDeviceMemoryConst(), (float const *)dy_buf.LockDeviceMemoryConst(), (float *)dx_buf.LockDeviceMemory(true), nullptr, idx,
                nullptr, this->m_W->DevConst(), this->m_dW->Dev(), 0, I, O, F, fs, 0, 0, this->m_binary_mode, this->m_lut_binarize,
                this->m_unbinarize_bias, st));
        return dx_buf;
    }

protected:
    void CommandProc(std::vector<std::string> const &args) override
    {
        Model::CommandProc(args);
        if (args.size() != 2) return;
        if (!kBit && args[0] == "binary") this->m_binary_mode = Model::EvalBool(args[1]);
        if (args[0] == "lut_binarize")    this->m_lut_binarize = Model::EvalBool(args[1]);
    }
};


// ---------------------------------------------------------------------------------------------------
// BinaryLutN<6, Bit>: bit-packed inference LUT (no backward), tables importable from a trained layer
// ---------------------------------------------------------------------------------------------------
template <int N = 6, typename FT = Bit, typename BT = float>
class BinaryLutN : public Model
{
    static_assert(N == 6 && std::is_same<FT, Bit>::value, "libbbcu_b200 implements BinaryLutN<6, Bit>");
    indices_t             m_input_shape, m_output_shape;
    Tensor_<std::int32_t> m_table;          // [node][2]: 64-entry truth table (BinaryLutN.h:43-46)
    Tensor_<std::int32_t> m_input_index;    // [node][6]
    std::string           m_connection;
    std::mt19937_64       m_mt;

public:
    struct create_t {
        indices_t     output_shape;
        std::string   connection;
        std::uint64_t seed = 1;
    };
    explicit BinaryLutN(create_t const &c) { m_output_shape = c.output_shape; m_connection = c.connection; m_mt.seed(c.seed); }
    static std::shared_ptr<BinaryLutN> Create(create_t const &c) { return std::make_shared<BinaryLutN>(c); }
    static std::shared_ptr<BinaryLutN> Create(index_t out, std::uint64_t seed = 1) { create_t c; c.output_shape = {out}; c.seed = seed; return Create(c); }
    static std::shared_ptr<BinaryLutN> CreatePy(indices_t output_shape, std::string connection = "", std::uint64_t seed = 1)
    {
        create_t c; c.output_shape = output_shape; c.connection = connection; c.seed = seed;
        return Create(c);
    }
    std::string GetModelName() const override { return "BinaryLut" + std::to_string(N); }
    std::string GetObjectName() const override { return GetModelName() + "_" + DataType<FT>::Name() + "_" + DataType<BT>::Name(); }

    // include/bb/BinaryLutN.h:481-520
    void DumpObjectData(std::ostream &os) const override
    {
        serial::Save(os, (std::int64_t)1);
        serial::SaveModelBase(os, this->m_name);
        serial::SaveBool(os, false);                         // host_only
        serial::SaveBool(os, true);                          // host_simd
        serial::SaveString(os, m_connection);
        serial::SaveShape(os, m_input_shape);
        serial::SaveShape(os, m_output_shape);
        serial::DumpTypedTensor(os, m_table);
        serial::DumpTypedTensor(os, m_input_index);
    }
    void LoadObjectData(std::istream &is) override
    {
        serial::ExpectVersion(is, 1, "BinaryLutN");
        this->m_name = serial::LoadModelBase(is);
        (void)serial::LoadBool(is);
        (void)serial::LoadBool(is);
        m_connection = serial::LoadString(is);
        m_input_shape  = serial::LoadShape(is);
        m_output_shape = serial::LoadShape(is);
        serial::LoadTypedTensor(is, m_table);
        serial::LoadTypedTensor(is, m_input_index);
        index_t I = CalcShapeSize(m_input_shape), O = CalcShapeSize(m_output_shape);
        if (m_table.GetShape() != indices_t({O, 2}) || m_input_index.GetShape() != indices_t({O, (index_t)N})) throw std::runtime_error("LoadObject: inconsistent layer shapes");
        std::int32_t const *t = m_input_index.HostConst();
        for (index_t i = 0; i < O * N; ++i)
            if (t[i] < 0 || t[i] >= I) throw std::runtime_error("LoadObject: connection index out of range");
    }
    indices_t GetInputShape()  const override { return m_input_shape; }
    indices_t GetOutputShape() const override { return m_output_shape; }

    indices_t SetInputShape(indices_t shape) override
    {
        if (shape == m_input_shape) return m_output_shape;
        m_input_shape = shape;
        index_t I = CalcShapeSize(shape), O = CalcShapeSize(m_output_shape);
        m_input_index.Resize({O, N});
        m_table.Resize({O, 2});
        // random wiring and random tables (include/bb/BinaryLutModel.h:31-58)
        ShuffleDeck deck(I, m_mt());
        auto idx = m_input_index.Host(true);
        for (index_t o = 0; o < O; ++o) { auto h = deck.Deal(N); for (int i = 0; i < N; ++i) idx[o * N + i] = (std::int32_t)h[i]; }
        std::mt19937_64 mt(m_mt());
        std::uniform_int_distribution<int> coin(0, 1);
        auto t = m_table.Host(true);
        for (index_t o = 0; o < O; ++o) {
            std::uint64_t bits = 0;
            for (int i = 0; i < 64; ++i) if (coin(mt)) bits |= (std::uint64_t)1 << i;
            t[o * 2] = (std::int32_t)(bits & 0xffffffffu); t[o * 2 + 1] = (std::int32_t)(bits >> 32);
        }
        return m_output_shape;
    }

    index_t GetNodeConnectionIndex(index_t node, index_t i) const { return m_input_index.HostConst()[node * N + i]; }
    void    SetNodeConnectionIndex(index_t node, index_t i, index_t in_node) { m_input_index.Host()[node * N + i] = (std::int32_t)in_node; }
    int     GetLutTableSize(index_t) const { return 64; }
    bool    GetLutTable(index_t node, int bitpos) const { return ((m_table.HostConst()[node * 2 + (bitpos >> 5)] >> (bitpos & 31)) & 1) != 0; }
    void    SetLutTable(index_t node, int bitpos, bool v)
    {
        auto &w = m_table.Host()[node * 2 + (bitpos >> 5)];
        std::uint32_t m = 1u << (bitpos & 31);
        w = (std::int32_t)(v ? ((std::uint32_t)w | m) : ((std::uint32_t)w & ~m));
    }

    // Freeze a trained sparse layer into truth tables: table[i] = (W[i] >= 0.5) (include/bb/BinaryLutModel.h:95-123)
    template <class SparseLayer>
    void ImportLayer(SparseLayer &src)
    {
        BB_ASSERT(src.GetOutputShape() == m_output_shape);
        SetInputShape(src.GetInputShape());
        index_t O = CalcShapeSize(m_output_shape);
        float const *W = src.W().HostConst();
        for (index_t o = 0; o < O; ++o) {
            for (int i = 0; i < N; ++i) SetNodeConnectionIndex(o, i, src.GetNodeConnectionIndex(o, i));
            for (int i = 0; i < 64; ++i) SetLutTable(o, i, W[o * 64 + i] >= 0.5f);
        }
    }

    FrameBuffer Forward(FrameBuffer x_buf, bool /*train*/ = true) override
    {
        BB_ASSERT(x_buf.GetType() == BB_TYPE_BIT);
        if (x_buf.GetShape() != m_input_shape) SetInputShape(x_buf.GetShape());
        FrameBuffer y_buf(x_buf.GetFrameSize(), m_output_shape, BB_TYPE_BIT);
        BBCU_CHECK(bbcu_bit_BinaryLut6_Forward((int const *)x_buf.LockDeviceMemoryConst(), (int *)y_buf.LockDeviceMemory(true), m_input_index.DevConst(),
                                               m_table.DevConst(), (int)y_buf.GetNodeSize(), (int)y_buf.GetFrameSize(),
                                               (int)(y_buf.GetFrameStride() / 4), Manager::Stream()));
        return y_buf;
    }
    FrameBuffer Backward(FrameBuffer dy_buf) override { return dy_buf.Empty() ? dy_buf : FrameBuffer(); }   // BinaryLutN.h:467-475: no backward
};


// ---------------------------------------------------------------------------------------------------
// StochasticBatchNormalization<float>
// ---------------------------------------------------------------------------------------------------
template <typename T = float>
class StochasticBatchNormalization : public Model
{
    indices_t m_shape;
    float m_momentum, m_gamma, m_beta;
    Tensor m_mean, m_rstd, m_running_mean, m_running_var;

public:
    struct create_t { float momentum = 0.9f, gamma = 0.2f, beta = 0.5f; };
    explicit StochasticBatchNormalization(create_t const &c) : m_momentum(c.momentum), m_gamma(c.gamma), m_beta(c.beta) {}
    static std::shared_ptr<StochasticBatchNormalization> Create(float momentum = 0.9f, float gamma = 0.2f, float beta = 0.5f)
    {
        create_t c; c.momentum = momentum; c.gamma = gamma; c.beta = beta;
        return std::make_shared<StochasticBatchNormalization>(c);
    }
    std::string GetModelName() const override { return "StochasticBatchNormalization"; }
    indices_t GetInputShape()  const override { return m_shape; }
    indices_t GetOutputShape() const override { return m_shape; }
    Tensor &running_mean() { return m_running_mean; }
    Tensor &running_var()  { return m_running_var; }
    Tensor &tmp_mean()     { return m_mean; }
    Tensor &tmp_rstd()     { return m_rstd; }

    indices_t SetInputShape(indices_t shape) override
    {
        if (shape == m_shape) return m_shape;
        m_shape = shape;
        index_t O = CalcShapeSize(shape);
        m_mean.Resize(O); m_rstd.Resize(O);
        m_running_mean.Resize(O); m_running_mean.Fill(0.0f);
        m_running_var.Resize(O);  m_running_var.Fill(1.0f);
        return m_shape;
    }

    FrameBuffer Forward(FrameBuffer x_buf, bool train = true) override
    {
        BB_ASSERT(x_buf.GetType() == BB_TYPE_FP32);
        if (x_buf.GetShape() != m_shape) SetInputShape(x_buf.GetShape());
        FrameBuffer y_buf(x_buf.GetFrameSize(), x_buf.GetShape(), BB_TYPE_FP32);
        if (train) PushFrameBuffer(x_buf);
        int O = (int)x_buf.GetNodeSize(), F = (int)x_buf.GetFrameSize(), s = (int)(x_buf.GetFrameStride() / 4);
        if (train) BBCU_CHECK(bbcu_fp32_StochasticBatchNormalization_ForwardTraining(
                (float const *)x_buf.LockDeviceMemoryConst(), (float *)y_buf.LockDeviceMemory(true), m_mean.Dev(true), m_rstd.Dev(true), m_running_mean.Dev(),
                m_running_var.Dev(), m_gamma, m_beta, m_momentum, O, F, s, Manager::Stream()));
        else BBCU_CHECK(bbcu_fp32_StochasticBatchNormalization_ForwardInference(
                (float const *)x_buf.LockDeviceMemoryConst(), (float *)y_buf.LockDeviceMemory(true), m_running_mean.DevConst(), m_running_var.DevConst(),
                m_gamma, m_beta, O, F, s, Manager::Stream()));
        return y_buf;
    }

    FrameBuffer ReForward(FrameBuffer x_buf)
    {
        FrameBuffer y_buf(x_buf.GetFrameSize(), x_buf.GetShape(), BB_TYPE_FP32);
        PushFrameBuffer(x_buf);
        BBCU_CHECK(bbcu_fp32_StochasticBatchNormalization_ReForward((float const *)x_buf.LockDeviceMemoryConst(), (float *)y_buf.LockDeviceMemory(true),
                                                                    m_mean.DevConst(), m_rstd.DevConst(), m_gamma, m_beta, (int)x_buf.GetNodeSize(),
                                                                    (int)x_buf.GetFrameSize(), (int)(x_buf.GetFrameStride() / 4), Manager::Stream()));
        return y_buf;
    }

    FrameBuffer Backward(FrameBuffer dy_buf) override
    {
        if (dy_buf.Empty()) return FrameBuffer();
        FrameBuffer dx_buf(dy_buf.GetFrameSize(), dy_buf.GetShape(), BB_TYPE_FP32);
        FrameBuffer x_buf = PopFrameBuffer();
        BBCU_CHECK(bbcu_fp32_StochasticBatchNormalization_Backward(
                (float const *)x_buf.LockDeviceMemoryConst(), (float const *)dy_buf.LockDeviceMemoryConst(), (float *)dx_buf.LockDeviceMemory(true),
                m_mean.DevConst(), m_rstd.DevConst(), m_gamma, 1.0f / (float)dy_buf.GetFrameSize(), (int)dy_buf.GetNodeSize(), (int)dy_buf.GetFrameSize(),
                (int)(dy_buf.GetFrameStride() / 4), (int)(x_buf.GetFrameStride() / 4), Manager::Stream()));
        return dx_buf;
    }

protected:
    void CommandProc(std::vector<std::string> const &args) override
    {
        Model::CommandProc(args);
        if (args.size() == 2 && args[0] == "set_gamma") m_gamma = std::stof(args[1]);
        if (args.size() == 2 && args[0] == "set_beta")  m_beta  = std::stof(args[1]);
        if (args.size() == 2 && args[0] == "momentum")  m_momentum = std::stof(args[1]);
    }
};


// ---------------------------------------------------------------------------------------------------
// OptimizerAdam<float> over a list of (parameter, gradient) tensors (include/bb/OptimizerAdam.h:47-184)
// ---------------------------------------------------------------------------------------------------
template <typename T = float>
class OptimizerAdam
{
    std::vector<std::shared_ptr<Tensor>> m_params, m_grads, m_m, m_v;
    Tensor_<std::int32_t> m_sizes;
    Tensor_<std::int64_t> m_ptab[4];
    float m_lr, m_beta1, m_beta2, m_b1, m_b2;

public:
    struct create_t { float learning_rate = 0.001f, beta1 = 0.9f, beta2 = 0.999f; };
    explicit OptimizerAdam(create_t const &c) : m_lr(c.learning_rate), m_beta1(c.beta1), m_beta2(c.beta2), m_b1(c.beta1), m_b2(c.beta2) {}
    static std::shared_ptr<OptimizerAdam> Create(float lr = 0.001f, float beta1 = 0.9f, float beta2 = 0.999f)
    {
        create_t c; c.learning_rate = lr; c.beta1 = beta1; c.beta2 = beta2;
        return std::make_shared<OptimizerAdam>(c);
    }
    void SetLearningRate(double lr) { m_lr = (float)lr; }

    void AddVariables(std::shared_ptr<Tensor> param, std::shared_ptr<Tensor> grad)
    {
        BB_ASSERT(param->GetShape() == grad->GetShape());
        m_params.push_back(param); m_grads.push_back(grad);
        auto m = std::make_shared<Tensor>(param->GetShape()), v = std::make_shared<Tensor>(param->GetShape());
        m->FillZero(); v->FillZero();
        m_m.push_back(m); m_v.push_back(v);
    }

    void Step()
    {
        if (m_params.empty()) return;
        int n = (int)m_params.size();
        m_sizes.Resize(n);
        for (auto &t : m_ptab) t.Resize(n);
        auto sz = m_sizes.Host(true);
        std::int64_t *p[4] = {m_ptab[0].Host(true), m_ptab[1].Host(true), m_ptab[2].Host(true), m_ptab[3].Host(true)};
        for (int i = 0; i < n; ++i) {
            sz[i] = (std::int32_t)m_params[i]->GetSize();
            p[0][i] = (std::int64_t)m_params[i]->Dev(); p[1][i] = (std::int64_t)m_grads[i]->Dev();
            p[2][i] = (std::int64_t)m_m[i]->Dev();      p[3][i] = (std::int64_t)m_v[i]->Dev();
        }
        float lr_t = m_lr * std::sqrt(1.0f - m_b2) / (1.0f - m_b1);
        BBCU_CHECK(bbcu_fp32_OptimizerAdam(n, m_sizes.DevConst(), (float *const *)m_ptab[0].DevConst(), (float *const *)m_ptab[1].DevConst(),
                                           (float *const *)m_ptab[2].DevConst(), (float *const *)m_ptab[3].DevConst(), lr_t, m_beta1, m_beta2,
                                           Manager::Stream()));
        m_b1 *= m_beta1;
        m_b2 *= m_beta2;
    }
    void ZeroGrad()
    {
        for (auto &g : m_grads) BBCU_CHECK(bbcu_fp32_Vector_set(g->Dev(true), 0.0f, (int)g->GetSize(), Manager::Stream()));
    }
    void Update() { Step(); ZeroGrad(); }      // include/bb/Optimizer.h:29-33
};

}   // namespace bb
