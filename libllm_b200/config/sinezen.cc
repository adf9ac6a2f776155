// The Sinezen decoder: its configuration and its description as parts.
//
// config.json (`architecture`: "Sinezen") lists the layers one by one.  Every layer is a parallel
// block, x + mixer(norm x) + ff(norm x) with one RMS norm, and names
//   type    the mixer; "attention": grouped-query attention with an RMS norm over the whole q and the
//           whole k projection before a partial half-split rotation, a score scale of its own, a
//           chunked mask (`mask.size`: a query sees the keys of its own block of that many
//           positions), values of a width of their own (`vdim`) and a sigmoid gate per head on the
//           heads' results;
//   mlp     null, {kind "dense", ff}: down(silu(gate h) * up h), or {kind "moe", router {experts,
//           top}, expert {ff}, shared {ff} or null}: experts down(gelu(up x)) chosen by the `top`
//           largest sigmoid(router h), each fed its score times h, plus a shared expert for all.
// `loop` {start, stop, times}: the layers from `start` up to, not including, `stop` are repeated
// `times` times and share their weights, while every repetition keeps a cache of its own; a
// repetition begins by replacing the stream with W_in [x; token rows] (tensor "loop.in").  Then the last norm ("final.norm") and the output
// matrix ("head").  Tensors of layer i are "l<i>.norm1", "l<i>.mix.{q,k,v,o,g,q.norm,k.norm}",
// "l<i>.mlp.{gate,up,down}" or "l<i>.mlp.{router,e<j>.up,e<j>.down,shared.up,shared.down}".
//
// Every size and constant comes from config.json; the description below is data for the generic
// model (parts/spec.h), and nothing else in the library knows this architecture.
#include "config/config.h"

namespace llm {

namespace {

const int64_t DEFAULT_MAX_POSITIONS = 1 << 20;   // the design states no limit; an engine's cache sets the real one

Json parse_mixer(const Json &layer, const std::string &where) {
  ConfigReader lr(layer, where);
  const std::string type = lr.string("type");
  if (type != "attention") lr.fail("mixer type '" + type + "' is not known (attention)");
  ConfigReader r(lr.object("mixer"), where + ": mixer");
  Json m = Json::object();
  const int64_t heads = r.integer("heads");
  const int64_t kv = r.integer_or("kv_heads", heads);
  if (heads % kv) r.fail("'heads' must be a multiple of 'kv_heads'");
  const int64_t dim = r.integer("dim");
  m.set("heads", heads);
  m.set("kv_heads", kv);
  m.set("dim", dim);
  m.set("vdim", r.integer_or("vdim", dim));
  m.set("scale", r.number("scale", false));
  if (r.present("mask")) {
    ConfigReader mr(r.object("mask"), where + ": mixer.mask");
    Json mask = Json::object();
    mask.set("size", mr.integer("size"));
    m.set("mask", mask);
  } else {
    m.set("mask", Json());
  }
  if (r.present("rot")) {
    ConfigReader rr(r.object("rot"), where + ": mixer.rot");
    Json rot = Json::object();
    const int64_t dims = rr.integer("dims", 0);
    if (dims % 2 || dims > dim) rr.fail("'dims' must be even and at most 'dim'");
    rot.set("base", rr.number("base"));
    rot.set("dims", dims);
    m.set("rot", rot);
  } else {
    m.set("rot", Json());
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
    ConfigReader er(r.object("expert"), where + ": mlp.expert");
    Json expert = Json::object();
    expert.set("ff", er.integer("ff"));
    m.set("expert", expert);
    if (r.present("shared")) {
      ConfigReader sr(r.object("shared"), where + ": mlp.shared");
      Json shared = Json::object();
      shared.set("ff", sr.integer("ff"));
      m.set("shared", shared);
    } else {
      m.set("shared", Json());
    }
  } else {
    r.fail("feed-forward kind '" + kind + "' is not known (dense, moe)");
  }
  return m;
}

// config.json as read -> normal form: the same layout with every optional key present.
Json parse_sinezen(const Json &data) {
  const std::string where = "config.json";
  ConfigReader r(data, where);
  Json c = Json::object();
  c.set("architecture", "Sinezen");
  c.set("vocab", r.integer("vocab"));
  c.set("width", r.integer("width"));
  Json norm = Json::object();
  norm.set("eps", ConfigReader(r.object("norm"), where + ": norm").number("eps"));
  c.set("norm", norm);
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
    if (start >= stop || stop > (int64_t)layers.size()) lr.fail("'start' < 'stop' <= number of layers is required");
    Json loop = Json::object();
    loop.set("start", start);
    loop.set("stop", stop);
    loop.set("times", times);
    c.set("loop", loop);
  } else {
    c.set("loop", Json());
  }
  c.set("max_positions", r.integer_or("max_positions", DEFAULT_MAX_POSITIONS));
  return c;
}

ModelSpec describe_sinezen(const Json &c) {
  const int64_t width = c.get("width").as_int();
  const double eps = c.get("norm").get("eps").as_number();
  auto norm = [&](const std::string &weight) {
    Json n = Json::object();
    n.set("kind", "rmsnorm");
    n.set("size", width);
    n.set("eps", eps);
    n.set("weight", weight);
    return n;
  };
  auto mlp = [&](int64_t ff, const std::string &activation, const std::string &prefix) {
    Json f = Json::object();
    f.set("kind", "mlp");
    f.set("hidden", width);
    f.set("intermediate", ff);
    f.set("activation", activation);
    f.set("up", prefix + "up");
    f.set("down", prefix + "down");
    return f;
  };
  ModelSpec s;
  s.name = "Sinezen";
  s.vocab_size = c.get("vocab").as_int();
  s.hidden = width;
  s.embedding = "embed";
  const Json &layers = c.get("layers");
  for (size_t i = 0; i < layers.size(); ++i) {
    const Json &l = layers.at(i);
    const Json &m = l.get("mixer");
    const std::string p = "l" + std::to_string(i) + ".";
    Json attn = Json::object();
    attn.set("kind", "attention");
    attn.set("hidden", width);
    attn.set("n_heads", m.get("heads"));
    attn.set("n_kv_heads", m.get("kv_heads"));
    attn.set("head_dim", m.get("dim"));
    attn.set("v_head_dim", m.get("vdim"));
    attn.set("scale", m.get("scale"));
    attn.set("window", Json());
    attn.set("block", m.get("mask").is_null() ? Json() : m.get("mask").get("size"));
    attn.set("bias", false);
    if (!m.get("rot").is_null() && m.get("rot").get("dims").as_int() > 0) {
      Json rope = Json::object();
      rope.set("kind", "rope");
      rope.set("head_dim", m.get("dim"));
      rope.set("rotary_dim", m.get("rot").get("dims"));
      rope.set("theta", m.get("rot").get("base"));
      rope.set("scaling", Json());
      attn.set("position", rope);
    } else {
      attn.set("position", Json());
    }
    Json qk = Json::object();
    qk.set("q", p + "mix.q.norm");
    qk.set("k", p + "mix.k.norm");
    qk.set("eps", eps);
    attn.set("qk_norm", qk);
    attn.set("head_gate", p + "mix.g");
    attn.set("q", p + "mix.q");
    attn.set("k", p + "mix.k");
    attn.set("v", p + "mix.v");
    attn.set("o", p + "mix.o");
    Json ff;
    const Json &f = l.get("mlp");
    if (!f.is_null() && f.get("kind").as_string() == "dense") {
      ff = Json::object();
      ff.set("kind", "swiglu");
      ff.set("hidden", width);
      ff.set("intermediate", f.get("ff"));
      ff.set("gate", p + "mlp.gate");
      ff.set("up", p + "mlp.up");
      ff.set("down", p + "mlp.down");
    } else if (!f.is_null()) {
      ff = Json::object();
      ff.set("kind", "moe");
      ff.set("hidden", width);
      ff.set("experts", f.get("router").get("experts"));
      ff.set("top", f.get("router").get("top"));
      ff.set("score", "sigmoid");
      ff.set("renormalize", false);
      ff.set("weight_on", "input");
      ff.set("router", p + "mlp.router");
      Json expert = Json::object();
      expert.set("intermediate", f.get("expert").get("ff"));
      expert.set("activation", "gelu");
      expert.set("up", p + "mlp.e{}.up");
      expert.set("down", p + "mlp.e{}.down");
      ff.set("expert", expert);
      ff.set("shared", f.get("shared").is_null() ? Json() : mlp(f.get("shared").get("ff").as_int(), "gelu", p + "mlp.shared."));
    }
    Json block = Json::object();
    block.set("kind", "parallel");
    block.set("norm", norm(p + "norm1"));
    block.set("mixer", attn);
    block.set("ff", ff);
    s.layers.push_back(block);
  }
  // the order of runs: layers before the loop, the looped ones `times` times, the rest
  const int n = (int)layers.size();
  const Json &loop = c.get("loop");
  if (loop.is_null()) {
    for (int i = 0; i < n; ++i) s.schedule.push_back({i, -1, ""});
  } else {
    const int start = (int)loop.get("start").as_int(), stop = (int)loop.get("stop").as_int();
    for (int i = 0; i < start; ++i) s.schedule.push_back({i, -1, ""});
    for (int64_t t = 0; t < loop.get("times").as_int(); ++t)
      for (int i = start; i < stop; ++i) s.schedule.push_back({i, -1, i == start ? "loop.in" : ""});
    for (int i = stop; i < n; ++i) s.schedule.push_back({i, -1, ""});
  }
  s.final_norm = norm("final.norm");
  s.head = "head";
  s.max_positions = c.get("max_positions").as_int();
  return s;
}

}  // namespace

void register_architecture_unlocked(Architecture arch);   // config/config.cc

void register_sinezen_architecture() {
  Architecture a;
  a.name = "Sinezen";
  a.parse = parse_sinezen;
  a.describe = describe_sinezen;
  register_architecture_unlocked(std::move(a));
}

}  // namespace llm
