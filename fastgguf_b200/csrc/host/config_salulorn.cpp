// The Salulorn decoder's config.json, and the model it describes as data.
//
// Keys: "architecture": "Salulorn"; "vocab", "width"; "norm": {"eps"}; "layers": a list, each
// {"type": "gla" | "attention" | "latent_attention", "mixer": {...}, "mlp": {"kind": "dense", "ff"} | null}; optional
// "loop": {"start", "stop", "times"}.
//   gla mixer               {"heads", "dim", "vdim", "tau"} (and, optionally, "decay_rank": else the checkpoint's shapes give it)
//   attention mixer         {"heads", "kv_heads", "dim", "vdim", "scale", "conv": taps, "mask": {"size"}, "rot": {"base", "dims"},
//                            "softcap"} - conv, mask, rot and softcap are each left out by a model that has none
//   latent_attention mixer  {"heads", "dim", "rot_dim", "vdim", "kv_rank", "q_rank", "scale",
//                            "rot": {"base", "dims", "scaling": {"factor", "original", "fast", "slow"}}}
// Every size and constant above comes from the file.  What the design itself fixes is written here once: every layer is a
// parallel block (one norm, the mixer and the feed-forward both read it and both add to the stream); norms multiply by their
// weight as stored; the dense feed-forward is SwiGLU; attention has biases on q, k, v, a norm over the whole of q and of k,
// adjacent rotary pairs and a sink per head; latent attention has a sink and a sigmoid output gate; the gla mixer scales q
// by dim^-0.5; the head is a matrix of its own.  With "loop", layers start .. stop - 1 run `times` times in a row, every pass
// with caches and states of its own, and in front of each pass (the first too) the stream becomes W_in [x; embedding output].
// Tensor names: embed, head, final.norm, loop.in, l<i>.norm1, l<i>.mix.*, l<i>.mlp.gate / up / down.
#include <cmath>

#include "config.hpp"

namespace fg {

static const std::string kSalulornName = "Salulorn";

static const Json *object_or_null(const Json &d, const std::string &key, const std::string &where) {
    const Json *v = d.find(key);
    if (!v || v->is_null()) return nullptr;
    if (!v->is_object()) fail(FG_E_CONFIG, where + ": '" + key + "' must be an object");
    return v;
}

class SalulornConfig : public ModelConfig {
public:
    struct Layer {
        std::string type;                       // "gla" | "attention" | "latent_attention"
        long long heads = 0, kv_heads = 0, dim = 0, vdim = 0;
        double tau = 1.0;                       // gla
        long long decay_rank = -1;
        long long taps = 0, window = 0;         // attention
        double softcap = 0.0, scale = 0.0;
        bool rotates = false;
        double rot_base = 0;
        long long rot_dims = 0;
        long long rot_dim = 0, kv_rank = 0, q_rank = 0;      // latent attention
        bool scaled = false;
        double factor = 1.0, original = 0.0, fast = 0.0, slow = 0.0;
        long long ff = 0;                       // 0: no feed-forward
    };
    Json source;
    long long vocab = 0, width = 0;
    double eps = 0.0;
    bool loops = false;
    long long loop_start = 0, loop_stop = 0, loop_times = 1;
    std::vector<Layer> layers;

    static std::unique_ptr<ModelConfig> from_json(const Json &d) {
        auto cfg = std::make_unique<SalulornConfig>();
        SalulornConfig &c = *cfg;
        c.source = d;
        c.vocab = take_int(d, "vocab");
        c.width = take_int(d, "width");
        const Json *norm = object_or_null(d, "norm", "config.json");
        if (!norm) fail(FG_E_CONFIG, "config.json: 'norm' must be an object");
        c.eps = take_float(*norm, "eps", "config.json norm");
        if (c.vocab <= 0 || c.width <= 0) fail(FG_E_CONFIG, "config.json: vocab and width must be positive");
        if (!(c.eps > 0.0)) fail(FG_E_CONFIG, format("config.json: norm.eps must be positive, got %g", c.eps));
        const Json *ls = d.find("layers");
        if (!ls || !ls->is_array() || ls->size() == 0) fail(FG_E_CONFIG, "config.json: 'layers' must be a non-empty list");
        for (size_t i = 0; i < ls->size(); i++) {
            const Json &l = (*ls)[i];
            std::string w = format("config.json layers[%zu]", i);
            if (!l.is_object()) fail(FG_E_CONFIG, w + " must be an object");
            Layer y;
            y.type = take_string(l, "type", "", w.c_str());
            const Json *mp = object_or_null(l, "mixer", w);
            if (!mp) fail(FG_E_CONFIG, w + ": 'mixer' must be an object");
            const Json &m = *mp;
            std::string wm = w + ".mixer";
            y.heads = take_int(m, "heads", wm.c_str());
            y.dim = take_int(m, "dim", wm.c_str());
            y.vdim = take_int(m, "vdim", y.dim, wm.c_str());
            if (y.heads <= 0 || y.dim <= 0 || y.vdim <= 0) fail(FG_E_CONFIG, wm + ": heads, dim and vdim must be positive");
            auto read_rot = [&](bool required) {
                const Json *rot = object_or_null(m, "rot", wm);
                if (!rot) {
                    if (required) fail(FG_E_CONFIG, wm + ": 'rot' must be an object");
                    return (const Json *)nullptr;
                }
                y.rotates = true;
                y.rot_base = take_float(*rot, "base", (wm + ".rot").c_str());
                if (!(y.rot_base > 1.0)) fail(FG_E_CONFIG, wm + ".rot: base must exceed 1");
                return rot;
            };
            if (y.type == "gla") {
                y.tau = take_float(m, "tau", 1.0, wm.c_str());
                y.decay_rank = take_int(m, "decay_rank", -1, wm.c_str());
                if (!(y.tau > 0.0)) fail(FG_E_CONFIG, wm + ": tau must be positive");
                if (y.decay_rank == 0 || y.decay_rank < -1) fail(FG_E_CONFIG, wm + ": decay_rank must be positive");
            } else if (y.type == "attention") {
                y.kv_heads = take_int(m, "kv_heads", y.heads, wm.c_str());
                if (y.kv_heads <= 0 || y.heads % y.kv_heads)
                    fail(FG_E_CONFIG, wm + format(": heads (%lld) must be a multiple of kv_heads (%lld)", y.heads, y.kv_heads));
                y.scale = take_float(m, "scale", 1.0 / std::sqrt((double)y.dim), wm.c_str());
                y.taps = take_int(m, "conv", 0, wm.c_str());
                y.softcap = take_float(m, "softcap", 0.0, wm.c_str());
                if (y.taps < 0 || y.softcap < 0.0) fail(FG_E_CONFIG, wm + ": conv and softcap cannot be negative");
                if (const Json *mask = object_or_null(m, "mask", wm)) {
                    y.window = take_int(*mask, "size", (wm + ".mask").c_str());
                    if (y.window <= 0) fail(FG_E_CONFIG, wm + ".mask: size must be positive");
                }
                if (const Json *rot = read_rot(false)) {
                    y.rot_dims = take_int(*rot, "dims", y.dim, (wm + ".rot").c_str());
                    if (y.rot_dims <= 0 || y.rot_dims % 2 || y.rot_dims > y.dim)
                        fail(FG_E_CONFIG, wm + format(".rot: dims must be even, positive and at most dim, got %lld", y.rot_dims));
                    if (y.dim % 2) fail(FG_E_CONFIG, wm + format(": a rotated head needs an even dim, got %lld", y.dim));
                }
            } else if (y.type == "latent_attention") {
                y.rot_dim = take_int(m, "rot_dim", wm.c_str());
                y.kv_rank = take_int(m, "kv_rank", wm.c_str());
                y.q_rank = take_int(m, "q_rank", wm.c_str());
                if (y.rot_dim <= 0 || y.rot_dim % 2 || y.kv_rank <= 0 || y.q_rank <= 0)
                    fail(FG_E_CONFIG, wm + ": rot_dim (even), kv_rank and q_rank must be positive");
                y.scale = take_float(m, "scale", 1.0 / std::sqrt((double)(y.dim + y.rot_dim)), wm.c_str());
                const Json *rot = read_rot(true);
                y.rot_dims = take_int(*rot, "dims", y.rot_dim, (wm + ".rot").c_str());
                if (y.rot_dims != y.rot_dim) fail(FG_E_CONFIG, wm + format(".rot: dims (%lld) must equal rot_dim (%lld)", y.rot_dims, y.rot_dim));
                if (const Json *sc = object_or_null(*rot, "scaling", wm + ".rot")) {
                    std::string ws = wm + ".rot.scaling";
                    y.scaled = true;
                    y.factor = take_float(*sc, "factor", ws.c_str());
                    y.original = take_float(*sc, "original", ws.c_str());
                    y.fast = take_float(*sc, "fast", ws.c_str());
                    y.slow = take_float(*sc, "slow", ws.c_str());
                    if (!(y.factor > 0.0) || !(y.original > 0.0) || !(y.fast > 0.0) || !(y.slow > 0.0)) fail(FG_E_CONFIG, ws + ": every number must be positive");
                }
            } else {
                fail(FG_E_CONFIG, w + ": type '" + y.type + "' is not known (known: gla, attention, latent_attention)");
            }
            if (const Json *mlp = object_or_null(l, "mlp", w)) {
                std::string wf = w + ".mlp";
                std::string kind = take_string(*mlp, "kind", "dense", wf.c_str());
                if (kind != "dense") fail(FG_E_CONFIG, wf + ": kind '" + kind + "' is not known (known: dense)");
                y.ff = take_int(*mlp, "ff", wf.c_str());
                if (y.ff <= 0) fail(FG_E_CONFIG, wf + ": ff must be positive");
            }
            c.layers.push_back(std::move(y));
        }
        if (const Json *loop = object_or_null(d, "loop", "config.json")) {
            c.loops = true;
            c.loop_start = take_int(*loop, "start", "config.json loop");
            c.loop_stop = take_int(*loop, "stop", "config.json loop");
            c.loop_times = take_int(*loop, "times", "config.json loop");
            if (c.loop_start < 0 || c.loop_stop <= c.loop_start || c.loop_stop > (long long)c.layers.size() || c.loop_times < 1)
                fail(FG_E_CONFIG, format("config.json loop: need 0 <= start < stop <= %zu and times >= 1", c.layers.size()));
        }
        return cfg;
    }

    long long layer_parameters(const Layer &y) const {
        long long n = width;
        if (y.type == "gla") n += width * (2 * y.heads * y.dim + 3 * y.heads * y.vdim) + y.vdim;      // without the low-rank pair of unknown size
        else if (y.type == "attention") n += width * (y.heads * y.dim + y.kv_heads * (y.dim + y.vdim) + y.heads * y.vdim) + y.heads;
        else n += width * (y.q_rank + y.kv_rank + y.rot_dim + 2 * y.heads * y.vdim) + y.q_rank * y.heads * (y.dim + y.rot_dim) + y.kv_rank * y.heads * (y.dim + y.vdim);
        return n + 3 * width * y.ff;
    }
    long long parameter_count() const {
        long long n = 2 * vocab * width + width + (loops ? 2 * width * width : 0);
        for (auto &y : layers) n += layer_parameters(y);
        return n;
    }
    // the layers in the order they run; true where the loop's input map stands in front
    std::vector<std::pair<long long, bool>> order() const {
        std::vector<std::pair<long long, bool>> o;
        const long long n = (long long)layers.size();
        if (!loops) {
            for (long long i = 0; i < n; i++) o.emplace_back(i, false);
            return o;
        }
        for (long long i = 0; i < loop_start; i++) o.emplace_back(i, false);
        for (long long t = 0; t < loop_times; t++)
            for (long long i = loop_start; i < loop_stop; i++) o.emplace_back(i, i == loop_start);
        for (long long i = loop_stop; i < n; i++) o.emplace_back(i, false);
        return o;
    }

    const std::string &architecture() const override { return kSalulornName; }
    Json to_json() const override { return source; }

    Json describe() const override {
        Json d = Json::object();
        d.set("vocab_size", vocab);
        d.set("hidden_size", width);
        d.set("num_hidden_layers", (long long)layers.size());
        d.set("layer_runs", (long long)order().size());
        d.set("norm_eps", eps);
        long long kv_numbers = 0, state_floats = 0;
        Json kinds = Json::array();
        for (auto &y : layers) kinds.push(y.type + "+" + (y.ff ? "dense" : "none"));
        for (auto &run : order()) {
            const Layer &y = layers[(size_t)run.first];
            if (y.type == "attention") { kv_numbers += y.kv_heads * (y.dim + y.vdim); state_floats += y.taps > 1 ? (y.taps - 1) * (y.heads * y.dim + y.kv_heads * (y.dim + y.vdim)) : 0; }
            else if (y.type == "latent_attention") kv_numbers += y.kv_rank + y.rot_dim;
            else state_floats += y.heads * y.dim * y.vdim;
        }
        d.set("layer_kinds", kinds);
        d.set("parameters", parameter_count());
        Json kvb = Json::object(), pb = Json::object();
        kvb.set("bfloat16", kv_numbers * 2);
        kvb.set("float32", kv_numbers * 4);
        pb.set("bfloat16", parameter_count() * 2);
        pb.set("float32", parameter_count() * 4);
        d.set("kv_bytes_per_token", kvb);
        d.set("parameter_bytes", pb);
        d.set("state_bytes_per_sequence", state_floats * 4);
        d.set("eos_token_ids", Json::array());
        d.set("defaulted", Json::array());
        return d;
    }

    Json spec() const override;
};

static Json make_part(const char *kind, Json params, Json tensors = Json::object()) {
    Json p = Json::object();
    p.set("kind", kind);
    p.set("params", std::move(params));
    p.set("tensors", std::move(tensors));
    return p;
}

Json SalulornConfig::spec() const {
    auto norm = [&](const std::string &name) {
        Json p = Json::object();
        p.set("size", width);
        p.set("eps", eps);
        Json t = Json::object();
        t.set("weight", name);
        return make_part("rmsnorm", p, t);
    };
    auto rope = [&](long long head_dim, long long rotary_dim, double base, const Layer *scaled) {
        Json rp = Json::object();
        rp.set("head_dim", head_dim);
        rp.set("theta", base);
        rp.set("rotary_dim", rotary_dim);
        rp.set("layout", "adjacent");
        if (scaled && scaled->scaled) {
            Json sc = Json::object();
            sc.set("rope_type", "yarn");
            sc.set("factor", scaled->factor);
            sc.set("original_max_position_embeddings", scaled->original);
            sc.set("beta_fast", scaled->fast);
            sc.set("beta_slow", scaled->slow);
            rp.set("scaling", sc);
        } else rp.set("scaling", Json());
        return make_part("rope", rp);
    };
    Json ls = Json::array(), schedule = Json::array();
    for (size_t i = 0; i < layers.size(); i++) {
        const Layer &y = layers[i];
        const std::string pre = format("l%zu.", i), mx = pre + "mix.";
        Json layer = Json::object();
        layer.set("block", "parallel");
        Json mp = Json::object(), mt = Json::object();
        mp.set("hidden_size", width);
        mp.set("n_heads", y.heads);
        mp.set("head_dim", y.dim);
        mp.set("v_head_dim", y.vdim);
        mp.set("eps", eps);
        if (y.type == "gla") {
            mp.set("tau", y.tau);
            mp.set("q_scale", 1.0 / std::sqrt((double)y.dim));
            if (y.decay_rank > 0) mp.set("decay_rank", y.decay_rank);
            for (const char *n : {"q", "k", "v", "g", "o"}) mt.set(std::string(n) + "_proj.weight", mx + n);
            mt.set("decay_down.weight", mx + "a1");
            mt.set("decay_up.weight", mx + "a2");
            mt.set("decay_up.bias", mx + "a2.b");
            mt.set("norm.weight", mx + "norm");
            layer.set("mixer", make_part("gated_linear_attention", mp, mt));
        } else if (y.type == "attention") {
            mp.set("n_kv_heads", y.kv_heads);
            mp.set("scale", y.scale);
            mp.set("window", y.window);
            mp.set("softcap", y.softcap);
            mp.set("conv_taps", y.taps);
            mp.set("bias", true);
            mp.set("sink", true);
            mp.set("qk_norm", "whole");
            mp.set("position", y.rotates ? rope(y.dim, y.rot_dims, y.rot_base, nullptr) : Json());
            for (const char *n : {"q", "k", "v"}) {
                mt.set(std::string(n) + "_proj.weight", mx + n);
                mt.set(std::string(n) + "_proj.bias", mx + n + ".b");
                if (y.taps > 0) mt.set(std::string(n) + "_conv.weight", mx + n + ".conv");
            }
            mt.set("q_norm.weight", mx + "q.norm");
            mt.set("k_norm.weight", mx + "k.norm");
            mt.set("sinks", mx + "sink");
            mt.set("o_proj.weight", mx + "o");
            layer.set("mixer", make_part("sink_attention", mp, mt));
        } else {
            mp.set("rot_dim", y.rot_dim);
            mp.set("kv_rank", y.kv_rank);
            mp.set("q_rank", y.q_rank);
            mp.set("scale", y.scale);
            mp.set("sink", true);
            mp.set("gate", true);
            mp.set("position", rope(y.rot_dim, y.rot_dim, y.rot_base, &y));
            mt.set("q_down.weight", mx + "dq");
            mt.set("q_down_norm.weight", mx + "dq.norm");
            mt.set("q_up.weight", mx + "uq");
            mt.set("kv_down.weight", mx + "dkv");
            mt.set("kv_down_norm.weight", mx + "dkv.norm");
            mt.set("k_up.weight", mx + "uk");
            mt.set("v_up.weight", mx + "uv");
            mt.set("sinks", mx + "sink");
            mt.set("g_proj.weight", mx + "g");
            mt.set("o_proj.weight", mx + "o");
            layer.set("mixer", make_part("latent_attention", mp, mt));
        }
        layer.set("mixer_norm", norm(pre + "norm1"));
        if (y.ff > 0) {
            Json fp = Json::object(), ft = Json::object();
            fp.set("hidden_size", width);
            fp.set("d_ff", y.ff);
            for (const char *n : {"gate", "up", "down"}) ft.set(std::string(n) + "_proj.weight", pre + "mlp." + n);
            layer.set("feed_forward", make_part("swiglu", fp, ft));
        } else layer.set("feed_forward", Json());
        ls.push(layer);
    }
    for (auto &run : order()) {
        Json r = Json::object();
        r.set("layer", run.first);
        r.set("cache_from", Json());
        if (run.second) r.set("reenter", true);
        schedule.push(r);
    }
    Json ep = Json::object(), hp = Json::object(), et = Json::object(), ht = Json::object();
    ep.set("vocab_size", vocab);
    ep.set("hidden_size", width);
    hp.set("vocab_size", vocab);
    hp.set("hidden_size", width);
    et.set("weight", "embed");
    ht.set("weight", "head");
    Json s = Json::object();
    s.set("hidden_size", width);
    s.set("vocab_size", vocab);
    s.set("max_positions", 1LL << 20);          // the design has no longest sequence; tables are built for what the cache holds
    s.set("embedding", make_part("embedding", ep, et));
    s.set("layers", ls);
    s.set("schedule", schedule);
    if (loops) {
        Json rp = Json::object(), rt = Json::object();
        rp.set("hidden_size", width);
        rt.set("weight", "loop.in");
        s.set("reentry", make_part("concat_linear", rp, rt));
    }
    s.set("final_norm", norm("final.norm"));
    s.set("head", make_part("lm_head", hp, ht));
    s.set("stop_token_ids", Json::array());
    s.set("ignored_tensors", Json::array());
    return s;
}

std::unique_ptr<ModelConfig> salulorn_config_from_json(const Json &d) { return SalulornConfig::from_json(d); }

}  // namespace fg
