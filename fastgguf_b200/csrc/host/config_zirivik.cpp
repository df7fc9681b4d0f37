// The Zirivik decoder's config.json, and the model it describes as data.
//
// Keys: "architecture": "Zirivik"; "vocab", "width"; "embedding": {"scale"}; "norm": {"eps"}; "logit_softcap";
// "layers": a list, each {"type": "retention" | "attention", "mixer": {...}, "mlp": {...} | null}:
//   retention mixer  {"heads", "dim", "vdim", "decay": [per head], "rot": {"base", "dims"}}
//   attention mixer  {"heads", "kv_heads", "dim", "vdim", "scale", "mask": {"size", "keep_first"}, "kv_from": j (optional)}
//   mlp              {"kind": "dense", "ff"}  or  {"kind": "moe", "expert": {"ff", "limit"}, "router": {"experts", "top"}}
// Every size and constant above comes from the file; what the design itself fixes is written here once: norms
// multiply by (1 + w), the dense feed-forward's activation is relu squared, the experts' gate uses sigmoid(1.702 g) and
// (up + 1), router scores are sigmoids that weight the expert's input, the head is the embedding table (without the
// embedding's scale), attention layers do not rotate, retention scales k by dim^-0.5.
// Tensor names: embed, final.norm, l<i>.norm1 / norm1b / norm2 / norm2b, l<i>.mix.q / k / v / g / o,
// l<i>.mlp.up / down, l<i>.mlp.router, l<i>.mlp.e<j>.gate / up / down.
#include <cmath>

#include "config.hpp"

namespace fg {

static const std::string kZirivikName = "Zirivik";

static const Json &object_of(const Json &d, const std::string &key, const std::string &where) {
    const Json *v = d.find(key);
    if (!v || !v->is_object()) fail(FG_E_CONFIG, where + ": '" + key + "' must be an object");
    return *v;
}

class ZirivikConfig : public ModelConfig {
public:
    struct Layer {
        std::string type;                       // "retention" | "attention"
        long long heads = 0, kv_heads = 0, dim = 0, vdim = 0;
        std::vector<double> decay;
        bool rotates = false;
        double rot_base = 0;
        long long rot_dims = 0;
        double scale = 0;
        long long window = 0, keep_first = 0, kv_from = -1;
        std::string mlp;                        // "" (none) | "dense" | "moe"
        long long ff = 0, experts = 0, top = 0;
        double limit = 0;
    };
    Json source;                                // the file as read: to_json gives it back
    long long vocab = 0, width = 0;
    double embedding_scale = 1.0, eps = 0.0, softcap = 0.0;
    std::vector<Layer> layers;

    static std::unique_ptr<ModelConfig> from_json(const Json &d) {
        auto cfg = std::make_unique<ZirivikConfig>();
        ZirivikConfig &c = *cfg;
        c.source = d;
        c.vocab = take_int(d, "vocab");
        c.width = take_int(d, "width");
        c.embedding_scale = take_float(object_of(d, "embedding", "config.json"), "scale", "config.json embedding");
        c.eps = take_float(object_of(d, "norm", "config.json"), "eps", "config.json norm");
        c.softcap = take_float(d, "logit_softcap");
        if (c.vocab <= 0 || c.width <= 0) fail(FG_E_CONFIG, "config.json: vocab and width must be positive");
        if (!(c.eps > 0.0)) fail(FG_E_CONFIG, format("config.json: norm.eps must be positive, got %g", c.eps));
        if (!(c.softcap > 0.0)) fail(FG_E_CONFIG, format("config.json: logit_softcap must be positive, got %g", c.softcap));
        const Json *ls = d.find("layers");
        if (!ls || !ls->is_array() || ls->size() == 0) fail(FG_E_CONFIG, "config.json: 'layers' must be a non-empty list");
        for (size_t i = 0; i < ls->size(); i++) {
            const Json &l = (*ls)[i];
            std::string w = format("config.json layers[%zu]", i);
            if (!l.is_object()) fail(FG_E_CONFIG, w + " must be an object");
            Layer y;
            y.type = take_string(l, "type", "", w.c_str());
            const Json &m = object_of(l, "mixer", w);
            std::string wm = w + ".mixer";
            y.heads = take_int(m, "heads", wm.c_str());
            y.dim = take_int(m, "dim", wm.c_str());
            y.vdim = take_int(m, "vdim", wm.c_str());
            if (y.heads <= 0 || y.dim <= 0 || y.vdim <= 0) fail(FG_E_CONFIG, wm + ": heads, dim and vdim must be positive");
            if (y.type == "retention") {
                const Json *dl = m.find("decay");
                if (!dl || !dl->is_array() || (long long)dl->size() != y.heads)
                    fail(FG_E_CONFIG, wm + format(": 'decay' must list one number for each of the %lld heads", y.heads));
                for (auto &v : dl->items()) {
                    if (!v.is_number() || v.is_bool()) fail(FG_E_CONFIG, wm + ": a decay must be a number, got " + json_repr(v));
                    y.decay.push_back(v.as_double());
                }
                const Json *rot = m.find("rot");
                if (rot && !rot->is_null()) {
                    if (!rot->is_object()) fail(FG_E_CONFIG, wm + ": 'rot' must be an object");
                    y.rotates = true;
                    y.rot_base = take_float(*rot, "base", (wm + ".rot").c_str());
                    y.rot_dims = take_int(*rot, "dims", (wm + ".rot").c_str());
                    if (y.rot_dims <= 0 || y.rot_dims % 2 || y.rot_dims > y.dim)
                        fail(FG_E_CONFIG, wm + format(".rot: dims must be even, positive and at most dim, got %lld", y.rot_dims));
                }
                if (y.dim % 2) fail(FG_E_CONFIG, wm + format(": dim must be even, got %lld", y.dim));
            } else if (y.type == "attention") {
                y.kv_heads = take_int(m, "kv_heads", wm.c_str());
                if (y.kv_heads <= 0 || y.heads % y.kv_heads)
                    fail(FG_E_CONFIG, wm + format(": heads (%lld) must be a multiple of kv_heads (%lld)", y.heads, y.kv_heads));
                y.scale = take_float(m, "scale", wm.c_str());
                const Json *mask = m.find("mask");
                if (mask && !mask->is_null()) {
                    if (!mask->is_object()) fail(FG_E_CONFIG, wm + ": 'mask' must be an object");
                    y.window = take_int(*mask, "size", (wm + ".mask").c_str());
                    y.keep_first = take_int(*mask, "keep_first", 0, (wm + ".mask").c_str());
                    if (y.window <= 0 || y.keep_first < 0) fail(FG_E_CONFIG, wm + ".mask: size must be positive and keep_first not negative");
                }
                const Json *from = m.find("kv_from");
                if (from && !from->is_null()) {
                    y.kv_from = take_int(m, "kv_from", wm.c_str());
                    if (y.kv_from < 0 || y.kv_from >= (long long)i) fail(FG_E_CONFIG, wm + format(": kv_from must name an earlier layer, got %lld", y.kv_from));
                    const Layer &o = c.layers[(size_t)y.kv_from];
                    if (o.type != "attention" || o.kv_from >= 0)
                        fail(FG_E_CONFIG, wm + format(": kv_from names layer %lld, which has no keys and values of its own", y.kv_from));
                    if (o.kv_heads != y.kv_heads || o.dim != y.dim || o.vdim != y.vdim)
                        fail(FG_E_CONFIG, wm + format(": layer %lld keeps keys and values of other sizes", y.kv_from));
                }
            } else {
                fail(FG_E_CONFIG, w + ": type '" + y.type + "' is not known (known: retention, attention)");
            }
            const Json *mlp = l.find("mlp");
            if (mlp && !mlp->is_null()) {
                if (!mlp->is_object()) fail(FG_E_CONFIG, w + ": 'mlp' must be an object or null");
                std::string wf = w + ".mlp";
                y.mlp = take_string(*mlp, "kind", "", wf.c_str());
                if (y.mlp == "dense") {
                    y.ff = take_int(*mlp, "ff", wf.c_str());
                } else if (y.mlp == "moe") {
                    const Json &ex = object_of(*mlp, "expert", wf), &ro = object_of(*mlp, "router", wf);
                    y.ff = take_int(ex, "ff", (wf + ".expert").c_str());
                    y.limit = take_float(ex, "limit", (wf + ".expert").c_str());
                    y.experts = take_int(ro, "experts", (wf + ".router").c_str());
                    y.top = take_int(ro, "top", (wf + ".router").c_str());
                    if (y.experts <= 0 || y.top <= 0 || y.top > y.experts) fail(FG_E_CONFIG, wf + ".router: need 0 < top <= experts");
                    if (!(y.limit > 0.0)) fail(FG_E_CONFIG, wf + ".expert: limit must be positive");
                } else {
                    fail(FG_E_CONFIG, wf + ": kind '" + y.mlp + "' is not known (known: dense, moe)");
                }
                if (y.ff <= 0) fail(FG_E_CONFIG, wf + ": ff must be positive");
            }
            c.layers.push_back(std::move(y));
        }
        return cfg;
    }

    long long parameter_count() const {
        long long n = vocab * width + width;
        for (auto &y : layers) {
            n += 2 * width;                                                       // the mixer's two norms
            if (y.type == "retention") n += width * (2 * y.heads * y.dim + 2 * y.heads * y.vdim) + y.heads * y.vdim * width;
            else n += width * y.heads * y.dim + y.heads * y.vdim * width + (y.kv_from < 0 ? width * y.kv_heads * (y.dim + y.vdim) : 0);
            if (y.mlp == "dense") n += 2 * width + 2 * width * y.ff;
            else if (y.mlp == "moe") n += 2 * width + y.experts * (3 * width * y.ff + width);
        }
        return n;
    }

    const std::string &architecture() const override { return kZirivikName; }
    Json to_json() const override { return source; }

    Json describe() const override {
        Json d = Json::object();
        d.set("vocab_size", vocab);
        d.set("hidden_size", width);
        d.set("num_hidden_layers", (long long)layers.size());
        d.set("embedding_scale", embedding_scale);
        d.set("norm_eps", eps);
        d.set("logit_softcap", softcap);
        long long kv_bytes = 0, state_floats = 0;
        Json kinds = Json::array();
        for (auto &y : layers) {
            kinds.push(y.type + (y.kv_from >= 0 ? "(shared)" : "") + "+" + (y.mlp.empty() ? "none" : y.mlp));
            if (y.type == "attention" && y.kv_from < 0) kv_bytes += y.kv_heads * (y.dim + y.vdim);
            if (y.type == "retention") state_floats += y.heads * y.dim * y.vdim;
        }
        d.set("layer_kinds", kinds);
        d.set("parameters", parameter_count());
        Json kvb = Json::object(), pb = Json::object();
        kvb.set("bfloat16", kv_bytes * 2);
        kvb.set("float32", kv_bytes * 4);
        pb.set("bfloat16", parameter_count() * 2);
        pb.set("float32", parameter_count() * 4);
        d.set("kv_bytes_per_token", kvb);
        d.set("parameter_bytes", pb);
        d.set("state_bytes_per_sequence", state_floats * 4);
        Json eos = Json::array();
        d.set("eos_token_ids", eos);
        d.set("defaulted", Json::array());
        return d;
    }

    Json spec() const override;
};

static Json part(const char *kind, Json params, Json tensors = Json::object()) {
    Json p = Json::object();
    p.set("kind", kind);
    p.set("params", std::move(params));
    p.set("tensors", std::move(tensors));
    return p;
}

// The model as data: sandwich blocks (a norm in front of and behind every sublayer), mixers and feed-forwards chosen
// layer by layer, one schedule entry per layer; a layer with kv_from reads the cache of that layer's entry.
Json ZirivikConfig::spec() const {
    auto norm = [&](const std::string &name) {
        Json p = Json::object();
        p.set("size", width);
        p.set("eps", eps);
        p.set("offset", 1.0);
        Json t = Json::object();
        t.set("weight", name);
        return part("rmsnorm", p, t);
    };
    Json ls = Json::array(), schedule = Json::array(), ignored = Json::array();
    for (size_t i = 0; i < layers.size(); i++) {
        const Layer &y = layers[i];
        std::string pre = format("l%zu.", i);
        Json layer = Json::object();
        layer.set("block", "sandwich");
        Json mp = Json::object(), mt = Json::object();
        mp.set("hidden_size", width);
        mp.set("n_heads", y.heads);
        mp.set("head_dim", y.dim);
        mp.set("v_head_dim", y.vdim);
        if (y.type == "retention") {
            Json dl = Json::array();
            for (double v : y.decay) dl.push(Json(v));
            mp.set("decay", dl);
            mp.set("eps", eps);
            mp.set("k_scale", 1.0 / std::sqrt((double)y.dim));
            if (y.rotates) {
                Json rp = Json::object();
                rp.set("head_dim", y.dim);
                rp.set("theta", y.rot_base);
                rp.set("rotary_dim", y.rot_dims);
                rp.set("layout", "halves");
                rp.set("scaling", Json());
                mp.set("position", part("rope", rp));
            } else mp.set("position", Json());
            for (const char *n : {"q", "k", "v", "g", "o"}) mt.set(std::string(n) + "_proj.weight", pre + "mix." + n);
            layer.set("mixer", part("retention", mp, mt));
        } else {
            mp.set("n_kv_heads", y.kv_heads);
            mp.set("scale", y.scale);
            mp.set("position", Json());
            mp.set("window", y.window);
            mp.set("keep_first", y.keep_first);
            mp.set("queries_only", y.kv_from >= 0);
            for (const char *n : {"q", "k", "v", "o"}) {
                if (y.kv_from >= 0 && (n[0] == 'k' || n[0] == 'v')) continue;
                mt.set(std::string(n) + "_proj.weight", pre + "mix." + n);
            }
            layer.set("mixer", part("gqa_attention", mp, mt));
        }
        layer.set("mixer_norm", norm(pre + "norm1"));
        layer.set("mixer_post_norm", norm(pre + "norm1b"));
        if (y.mlp.empty()) {
            layer.set("feed_forward", Json());
        } else {
            Json fp = Json::object(), ft = Json::object();
            fp.set("hidden_size", width);
            fp.set("d_ff", y.ff);
            if (y.mlp == "dense") {
                fp.set("activation", "relu2");
                ft.set("up_proj.weight", pre + "mlp.up");
                ft.set("down_proj.weight", pre + "mlp.down");
                layer.set("feed_forward", part("mlp", fp, ft));
            } else {
                fp.set("n_experts", y.experts);
                fp.set("top_k", y.top);
                fp.set("limit", y.limit);
                fp.set("alpha", 1.702);
                fp.set("router", "sigmoid_input");
                ft.set("router.weight", pre + "mlp.router");
                for (long long e = 0; e < y.experts; e++)
                    for (const char *n : {"gate", "up", "down"})
                        ft.set(format("experts.%lld.%s_proj.weight", e, n), pre + format("mlp.e%lld.%s", e, n));
                layer.set("feed_forward", part("moe", fp, ft));
            }
            layer.set("feed_forward_norm", norm(pre + "norm2"));
            layer.set("feed_forward_post_norm", norm(pre + "norm2b"));
        }
        ls.push(layer);
        Json run = Json::object();
        run.set("layer", (long long)i);
        run.set("cache_from", y.kv_from >= 0 ? Json(y.kv_from) : Json());
        schedule.push(run);
    }
    Json ep = Json::object(), hp = Json::object(), et = Json::object();
    ep.set("vocab_size", vocab);
    ep.set("hidden_size", width);
    ep.set("scale", embedding_scale);
    hp.set("vocab_size", vocab);
    hp.set("hidden_size", width);
    hp.set("softcap", softcap);
    et.set("weight", "embed");
    Json s = Json::object();
    s.set("hidden_size", width);
    s.set("vocab_size", vocab);
    s.set("max_positions", 1LL << 20);          // the design has no longest sequence; tables are built for what the cache holds
    s.set("embedding", part("embedding", ep, et));
    s.set("layers", ls);
    s.set("schedule", schedule);
    s.set("final_norm", norm("final.norm"));
    s.set("head", part("lm_head", hp, et));
    s.set("stop_token_ids", Json::array());
    s.set("ignored_tensors", ignored);
    return s;
}

std::unique_ptr<ModelConfig> zirivik_config_from_json(const Json &d) { return ZirivikConfig::from_json(d); }

}  // namespace fg
