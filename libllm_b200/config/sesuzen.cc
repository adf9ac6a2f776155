// The Sesuzen decoder: its configuration and its description as parts.
//
// config.json (`architecture`: "Sesuzen") lists the layers one by one; every size and constant is
// read from it (or, for the rank of the decay's low-rank input, from the stored tensor).  The
// stream starts as token row + a learned vector per position ("embed", "pos").  Every layer is a
// pre-norm block, x += mixer(conv(norm1 x)), x += ff(norm2 x): layer norms with weight and bias
// ("l<i>.norm1", "l<i>.norm1.b"), and before the mixer a causal convolution over time per channel
// whose result is added to its input ("l<i>.canon1" [width, canon.taps]).  A layer names
//   type   "attention": grouped-query attention without a rotation, biases on q, k, v (".b"), every
//          value head divided by its root mean square before it is cached, a score scale of its
//          own, a sliding window (`mask.size`) that also keeps the first `mask.keep_first`
//          positions, and a sigmoid gate per channel on the concatenated heads ("mix.g");
//          "general_delta": the generalized delta rule (parts/recurrent.cc), tensors
//          "mix.{r,k,v,g,a,a.b,w1,w2,w0,norm,o}";
//   mlp    null, {kind "dense", ff}: down(relu(up h)^2), or {kind "moe", router {experts, top},
//          expert {ff}}: experts down(silu(gate h) * up h) chosen by the `top` largest router
//          logits, weighted by the softmax over the chosen logits.
// `loop` {start, stop, times}: layers start .. stop-1 run `times` times in a row with the same
// weights, each pass with a cache and state of its own.  Then the last layer norm ("final.norm"),
// the token table as output matrix, and logits bounded by logit_softcap * tanh(logits / logit_softcap).
#include <cmath>

#include "config/config.h"

namespace llm {

namespace {

Json parse_mixer(const Json &layer, const std::string &where) {
  ConfigReader lr(layer, where);
  const std::string type = lr.string("type");
  ConfigReader r(lr.object("mixer"), where + ": mixer");
  Json m = Json::object();
  const int64_t heads = r.integer("heads"), dim = r.integer("dim");
  m.set("heads", heads);
  m.set("dim", dim);
  if (type == "attention") {
    const int64_t kv = r.integer_or("kv_heads", heads);
    if (heads % kv) r.fail("'heads' must be a multiple of 'kv_heads'");
    m.set("kv_heads", kv);
    m.set("vdim", r.integer_or("vdim", dim));
    m.set("scale", r.number("scale", false));
    if (r.present("mask")) {
      ConfigReader mr(r.object("mask"), where + ": mixer.mask");
      Json mask = Json::object();
      mask.set("size", mr.integer("size"));
      mask.set("keep_first", mr.integer_or("keep_first", 0, 0));
      m.set("mask", mask);
    } else {
      m.set("mask", Json());
    }
  } else if (type == "general_delta") {
    m.set("rank", r.present("rank") ? Json(r.integer("rank")) : Json());      // null: the size "mix.w1" is stored with
  } else {
    lr.fail("mixer type '" + type + "' is not known (attention, general_delta)");
  }
  return m;
}

Json parse_mlp(const Json &raw, const std::string &where) {
  if (raw.is_null()) return Json();
  if (!raw.is_object()) LLM_THROW(Config, "%s: 'mlp' must be an object or null", where.c_str());
  ConfigReader r(raw, where + ": mlp");
  const std::string kind = r.string("kind");
  Json m = Json::object();
  m.set("kind", kind);
  if (kind == "dense") {
    m.set("ff", r.integer("ff"));
  } else if (kind == "moe") {
    ConfigReader rr(r.object("router"), where + ": mlp.router");
    Json router = Json::object();
    const int64_t experts = rr.integer("experts"), top = rr.integer("top");
    if (top > experts) rr.fail("'top' exceeds 'experts'");
    router.set("experts", experts);
    router.set("top", top);
    m.set("router", router);
    Json expert = Json::object();
    expert.set("ff", ConfigReader(r.object("expert"), where + ": mlp.expert").integer("ff"));
    m.set("expert", expert);
  } else {
    r.fail("feed-forward kind '" + kind + "' is not known (dense, moe)");
  }
  return m;
}

// config.json as read -> normal form: the same layout with every optional key present.
Json parse_sesuzen(const Json &data) {
  const std::string where = "config.json";
  ConfigReader r(data, where);
  Json c = Json::object();
  c.set("architecture", "Sesuzen");
  c.set("vocab", r.integer("vocab"));
  c.set("width", r.integer("width"));
  c.set("max_positions", r.integer("max_positions"));
  Json norm = Json::object();
  norm.set("eps", ConfigReader(r.object("norm"), where + ": norm").number("eps"));
  c.set("norm", norm);
  Json canon = Json::object();
  canon.set("taps", r.present("canon") ? ConfigReader(r.object("canon"), where + ": canon").integer("taps") : 0);
  c.set("canon", canon);
  c.set("logit_softcap", r.number_or("logit_softcap", 0.0, false));
  const Json &layers = data.get("layers");
  if (!layers.is_array() || layers.size() == 0) r.fail("'layers' must be a list with at least one layer");
  Json ls = Json::array();
  for (size_t i = 0; i < layers.size(); ++i) {
    const std::string lw = where + ": layers[" + std::to_string(i) + "]";
    const Json &l = layers.at(i);
    if (!l.is_object()) LLM_THROW(Config, "%s must be an object", lw.c_str());
    Json o = Json::object();
    o.set("type", ConfigReader(l, lw).string("type"));
    o.set("mixer", parse_mixer(l, lw));
    o.set("mlp", parse_mlp(l.get("mlp"), lw));
    ls.push(o);
  }
  c.set("layers", ls);
  if (r.present("loop")) {
    ConfigReader lr(r.object("loop"), where + ": loop");
    const int64_t start = lr.integer("start", 0), stop = lr.integer("stop", 0), times = lr.integer("times");
    if (start > stop || stop > (int64_t)layers.size()) lr.fail("'start' <= 'stop' <= number of layers is required");
    Json loop = Json::object();
    loop.set("start", start);
    loop.set("stop", stop);
    loop.set("times", times);
    c.set("loop", loop);
  } else {
    c.set("loop", Json());
  }
  return c;
}

ModelSpec describe_sesuzen(const Json &c) {
  const int64_t width = c.get("width").as_int();
  const double eps = c.get("norm").get("eps").as_number();
  const int64_t taps = c.get("canon").get("taps").as_int();
  auto norm = [&](const std::string &weight) {
    Json n = Json::object();
    n.set("kind", "layernorm");
    n.set("size", width);
    n.set("eps", eps);
    n.set("weight", weight);
    n.set("bias", weight + ".b");
    return n;
  };
  ModelSpec s;
  s.name = "Sesuzen";
  s.vocab_size = c.get("vocab").as_int();
  s.hidden = width;
  s.embedding = "embed";
  s.position_table = "pos";
  s.max_positions = c.get("max_positions").as_int();
  s.logit_softcap = c.get("logit_softcap").as_number();
  const Json &layers = c.get("layers");
  for (size_t i = 0; i < layers.size(); ++i) {
    const Json &l = layers.at(i);
    const Json &m = l.get("mixer");
    const std::string p = "l" + std::to_string(i) + ".", x = p + "mix.";
    Json mixer = Json::object();
    if (l.get("type").as_string() == "attention") {
      mixer.set("kind", "attention");
      mixer.set("hidden", width);
      mixer.set("n_heads", m.get("heads"));
      mixer.set("n_kv_heads", m.get("kv_heads"));
      mixer.set("head_dim", m.get("dim"));
      mixer.set("v_head_dim", m.get("vdim"));
      mixer.set("scale", m.get("scale"));
      mixer.set("position", Json());
      const Json &mask = m.get("mask");
      mixer.set("window", mask.is_null() ? Json() : mask.get("size"));
      if (!mask.is_null() && mask.get("keep_first").as_int() > 0) mixer.set("sink", mask.get("keep_first"));
      mixer.set("bias", true);
      mixer.set("q_bias", x + "q.b");
      mixer.set("k_bias", x + "k.b");
      mixer.set("v_bias", x + "v.b");
      Json vn = Json::object();
      vn.set("eps", eps);
      mixer.set("v_norm", vn);
      mixer.set("out_gate", x + "g");
      mixer.set("q", x + "q");
      mixer.set("k", x + "k");
      mixer.set("v", x + "v");
      mixer.set("o", x + "o");
    } else {
      mixer.set("kind", "general_delta");
      mixer.set("hidden", width);
      mixer.set("n_heads", m.get("heads"));
      mixer.set("head_dim", m.get("dim"));
      mixer.set("decay_rank", m.get("rank"));
      mixer.set("eps", eps);
      mixer.set("decay_scale", std::exp(-0.5));       // the design's constants: w = exp(-e^(-1/2) sigmoid(.)) ...
      mixer.set("key_eps", 1e-6);                      // ... and u = k / sqrt(sum k^2 + 1e-6)
      for (const char *t : {"r", "k", "v", "g", "a", "w1", "w2", "w0", "norm", "o"}) mixer.set(t, x + t);
      mixer.set("a_bias", x + "a.b");
    }
    Json ff;
    const Json &f = l.get("mlp");
    if (!f.is_null() && f.get("kind").as_string() == "dense") {
      ff = Json::object();
      ff.set("kind", "mlp");
      ff.set("hidden", width);
      ff.set("intermediate", f.get("ff"));
      ff.set("activation", "relu2");
      ff.set("up", p + "mlp.up");
      ff.set("down", p + "mlp.down");
    } else if (!f.is_null()) {
      ff = Json::object();
      ff.set("kind", "moe");
      ff.set("hidden", width);
      ff.set("experts", f.get("router").get("experts"));
      ff.set("top", f.get("router").get("top"));
      ff.set("score", "softmax");                      // softmax over all, divided by the chosen ones' sum:
      ff.set("renormalize", true);                     // the softmax over the chosen logits alone
      ff.set("weight_on", "output");
      ff.set("router", p + "mlp.router");
      Json expert = Json::object();
      expert.set("intermediate", f.get("expert").get("ff"));
      expert.set("activation", "silu");
      expert.set("gate", p + "mlp.e{}.gate");
      expert.set("up", p + "mlp.e{}.up");
      expert.set("down", p + "mlp.e{}.down");
      ff.set("expert", expert);
    }
    Json block = Json::object();
    block.set("kind", "prenorm");
    block.set("mixer_norm", norm(p + "norm1"));
    if (taps > 0) {
      Json conv = Json::object();
      conv.set("taps", taps);
      conv.set("weight", p + "canon1");
      conv.set("hidden", width);
      block.set("mixer_conv", conv);
    }
    block.set("mixer", mixer);
    block.set("ff_norm", ff.is_null() ? Json() : norm(p + "norm2"));
    block.set("ff", ff);
    s.layers.push_back(block);
  }
  const int n = (int)layers.size();
  const Json &loop = c.get("loop");
  if (loop.is_null()) {
    for (int i = 0; i < n; ++i) s.schedule.push_back({i, -1, ""});
  } else {
    const int start = (int)loop.get("start").as_int(), stop = (int)loop.get("stop").as_int();
    for (int i = 0; i < start; ++i) s.schedule.push_back({i, -1, ""});
    for (int64_t t = 0; t < loop.get("times").as_int(); ++t)
      for (int i = start; i < stop; ++i) s.schedule.push_back({i, -1, ""});
    for (int i = stop; i < n; ++i) s.schedule.push_back({i, -1, ""});
  }
  s.final_norm = norm("final.norm");
  s.head = "";                                        // the token table is the output matrix
  return s;
}

}  // namespace

void register_architecture_unlocked(Architecture arch);   // config/config.cc

void register_sesuzen_architecture() {
  Architecture a;
  a.name = "Sesuzen";
  a.parse = parse_sesuzen;
  a.describe = describe_sesuzen;
  register_architecture_unlocked(std::move(a));
}

}  // namespace llm
