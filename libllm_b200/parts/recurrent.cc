// Mixers that carry a fixed-size state from token to token instead of keys and values.
//
// "general_delta": the generalized delta rule.  Per head, with h the mixer's input and d channels:
//   r = W_r h, k = W_k h, v = W_v h
//   decay    w = exp(-decay_scale * sigmoid(w0 + W_2 tanh(W_1 h)))     per key channel (W_1 of low rank)
//   removal  a = sigmoid(W_a h + a_bias)                               per key channel
//   unit key u = k / sqrt(sum(k^2) + key_eps)
//   state    S <- diag(w) S - (a * u)(u^T S) + k v^T                   both terms read the old S
//   result   o = S^T r, divided by its root mean square over the head (eps), times `norm`
//            (a weight over all heads' channels), times sigmoid(W_g h), then W_o.
// The state (heads x d x d, 32-bit) starts at zero and belongs to the run and the sequence.  All
// projections of h are one stacked product [r; k; v; g; a; W_1] with a 32-bit result; everything
// from there to the state is 32-bit (csrc/recurrent.cu).  The reference has no such mixer.
#include <cmath>

#include "config/config.h"
#include "csrc/kernels.h"
#include "parts/chain.h"
#include "parts/linear.h"
#include "parts/part.h"

namespace llm {

namespace {

class GeneralDelta : public Mixer {
 public:
  GeneralDelta(const Json &spec, const BuildEnv &env) : Mixer(spec, env) {
    ConfigReader r(spec, "general_delta description");
    hidden_ = r.integer("hidden");
    n_heads_ = (int)r.integer("n_heads");
    d_ = (int)r.integer("head_dim");
    if (d_ > 256) LLM_THROW(Unsupported, "general_delta: heads of %d channels are not supported (up to 256)", d_);
    rank_ = r.integer_or("decay_rank", -1);          // -1: the size W_1 is stored with
    eps_ = (float)r.number("eps");
    decay_scale_ = (float)r.number_or("decay_scale", std::exp(-0.5));
    key_eps_ = (float)r.number_or("key_eps", 1e-6);
    for (const char *key : {"r", "k", "v", "g", "a", "a_bias", "w1", "w2", "w0", "norm", "o"}) names_.push_back(r.string(key));
    width_ = (int64_t)n_heads_ * d_;
  }
  enum { R, K, V, G, A, A_BIAS, W1, W2, W0, NORM, O };

  std::vector<TensorNeed> tensor_needs() const override {
    std::vector<TensorNeed> needs;
    for (int i : {R, K, V, G, A}) needs.push_back({names_[(size_t)i], {width_, hidden_}});
    needs.push_back({names_[A_BIAS], {width_}, TensorRole::Vector, false});
    needs.push_back({names_[W1], {rank_, hidden_}});
    needs.push_back({names_[W2], {width_, rank_}, TensorRole::Vector, false});
    needs.push_back({names_[W0], {width_}, TensorRole::Vector, false});
    needs.push_back({names_[NORM], {width_}, TensorRole::Vector, false});
    needs.push_back({names_[O], {hidden_, width_}});
    return needs;
  }

  void load(const Loader &l) override {
    if (rank_ < 0) {
      const std::vector<int64_t> stored = l.shape_of(names_[W1]);
      rank_ = stored.size() == 2 ? stored[0] : DRAWN_FREE_SIZE;
    }
    const std::vector<TensorNeed> needs = tensor_needs();
    const size_t es = dtype_size(l.engine);
    // rows of the stacked matrix in multiples of 8, so that rows of the 32-bit product start on 32 bytes
    w_in_.dtype = l.engine;
    w_in_.rows = (5 * width_ + rank_ + 7) / 8 * 8;
    w_in_.cols = hidden_;
    w_in_.buf.allocate((size_t)w_in_.rows * (size_t)hidden_ * es, true);
    for (int i = 0; i < 5; ++i) l.fetch_into(needs[(size_t)i], l.engine, (char *)w_in_.buf.get() + (size_t)i * width_ * hidden_ * es);
    l.fetch_into(needs[6], l.engine, (char *)w_in_.buf.get() + (size_t)5 * width_ * hidden_ * es);
    a_bias_ = l.fetch(needs[5]);
    w2_ = l.fetch(needs[7]);
    w0_ = l.fetch(needs[8]);
    norm_ = l.fetch(needs[9]);
    w_o_ = l.fetch(needs[10]);
  }

  std::vector<std::string> kernel_families() const override {
    std::vector<std::string> fams = product_families(env_.dtype);
    fams.push_back("recurrent");
    return fams;
  }

  std::vector<StateNeed> state_need() const override { return {{"general_delta.S", {(int64_t)n_heads_, (int64_t)d_, (int64_t)d_}, DType::F32}}; }

  Act forward(StepContext &ctx, const Act &x, LayerCache *, StateView *state) override {
    float *S = nullptr;
    if (state)
      for (const auto &t : *state)
        if (t.name == "general_delta.S") S = (float *)t.data;
    if (!S) LLM_THROW(InvalidArg, "general_delta: the run has no state");
    Act proj = linear(ctx, x, w_in_, nullptr, DType::F32);
    flush_chain(ctx);
    const int T = ctx.n_tokens;
    const int W = (int)width_;
    if (ctx.decode_only && T == ctx.n_seqs && kernels::delta_step_supported(d_)) {
      // a step of single tokens: the vectors, the state's step, the norm and the gate in one launch
      Act y = ctx.arena->act(ctx.dtype, T, width_);
      kernels::delta_step(proj, 0, W, 2 * W, 3 * W, 4 * W, 5 * W, (int)rank_, w2_.buf.as<float>(), w0_.buf.as<float>(),
                          a_bias_.buf.as<float>(), decay_scale_, key_eps_, norm_.buf.as<float>(), eps_, S, y, ctx.seq_slot, n_heads_, d_,
                          ctx.stream);
      return linear(ctx, y, w_o_, nullptr, DType::F32, true);
    }
    float *prep = ctx.arena->alloc_n<float>((size_t)T * (size_t)width_ * 3);
    Act o = ctx.arena->act(DType::F32, T, width_);
    kernels::delta_rule(proj, 0, W, 2 * W, 4 * W, 5 * W, (int)rank_, w2_.buf.as<float>(), w0_.buf.as<float>(), a_bias_.buf.as<float>(),
                        decay_scale_, key_eps_, prep, S, o, ctx.seq_start, ctx.seq_slot, ctx.n_seqs, n_heads_, d_, ctx.stream);
    Act y = ctx.arena->act(ctx.dtype, T, width_);
    kernels::head_norm_gate(o, norm_.buf.as<float>(), (const float *)proj.data + 3 * W, proj.ld, eps_, n_heads_, d_, y, ctx.stream);
    return linear(ctx, y, w_o_, nullptr, DType::F32, true);
  }

 private:
  int64_t hidden_, width_, rank_;
  int n_heads_, d_;
  float eps_, decay_scale_, key_eps_;
  std::vector<std::string> names_;
  Weight w_in_, w_o_, a_bias_, w2_, w0_, norm_;
};

}  // namespace

void register_part_raw(const std::string &category, const std::string &kind, PartFactory factory);   // parts/part.cc

void register_recurrent_parts() {
  register_part_raw("mixer", "general_delta",
                    [](const Json &spec, const BuildEnv &env) { return std::unique_ptr<Part>(new GeneralDelta(spec, env)); });
}

}  // namespace llm
