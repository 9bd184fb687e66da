// Parallel-block families (Punilix, Gamanex) and the sequential-sublayer families (Vugipel, Vakesun) inside the host engine: configuration, weights, scratch and the encoding of one pass.
// Included by engine.cu; the pass driver, the state / cache manager, sampling, CUDA-graph decode and the sequence slots are the engine's own.
//
//   x = embed[token]                                                      (f32 residual stream)
//   Punilix layer:  h = group_rms(x);  x <- x + mixer(h) + mlp(h)         (one norm feeds both sublayers)
//   Gamanex layer:  h1 = rms(x) n1, h2 = rms(x) n2;  x <- x + ls1 sigmoid(G1 h1 + b1) mixer(h1) + ls2 sigmoid(G2 h2 + b2) mlp(h2)
//   Vugipel layer:  x <- x + mixer(rms(x) (1 + n1));  x <- x + mlp(rms(x) (1 + n2))     (Layer::sequential)
//   Vakesun layer:  x <- x + m post1(mixer(pre1(x)));  x <- x + m post2(mlp(pre2(x)));  x <- x + m rms(token input(x))    (Layer::sandwich)
//   logits = cap * tanh(head . group_rms(x) / cap)   |   logit_scale * head . rms(x)
//
// Both are described by the same Layer fields (a second norm, sublayer gates and a logit scale are optional parts) and encoded by the same
// loop; a family is a config reader that fills them.
// config.json: "architecture", "width", "vocab", "norm": {"eps", "groups"}, "logit_softcap" | "logit_scale", "layers": [{"type", "mixer": {...}, "mlp"}].
// Tensors: embed, head, final.norm, l<i>.norm1 (norm2), l<i>.mix.*, l<i>.mlp.* (bf16 or f32 floats, i32 tables); linear weights are [out, in].
// Weights are assembled on the host at load: projections that read the same input are stacked into one matrix, per-head key
// up-projections are transposed for the absorbed form, expert matrices lie back to back. Storage is bf16, or f32 when the engine was
// created with storage_f32 (then every product is a plain f32 multiply-add).

namespace {

struct HostTensor {
    std::vector<float> v;
    std::vector<uint64_t> shape;
    uint64_t rows() const { return shape.empty() ? 0 : shape[0]; }
    uint64_t cols() const { return shape.size() < 2 ? 1 : shape[1]; }
};

static HostTensor read_floats(ParameterLoader& pl, const std::string& name, const std::vector<uint64_t>& shape) {
    auto it = pl.tensors.find(name);
    if (it == pl.tensors.end()) throw std::runtime_error("missing tensor '" + name + "'");
    const std::string dt = it->second.dtype;
    if (dt != "BF16" && dt != "F32") throw std::runtime_error("tensor '" + name + "' has dtype " + dt + ", expected BF16 or F32");
    const TensorInfo& t = pl.validate(name, shape, dt);
    HostTensor h;
    h.shape = shape;
    uint64_t n = 1;
    for (auto d : shape) n *= d;
    h.v.resize(n);
    if (dt == "F32") {
        pl.read_into(t, h.v.data());
    } else {
        std::vector<uint16_t> raw(n);
        pl.read_into(t, raw.data());
        for (uint64_t i = 0; i < n; ++i) {
            const uint32_t bits = (uint32_t)raw[i] << 16;
            memcpy(&h.v[i], &bits, 4);
        }
    }
    return h;
}

static uint16_t f32_to_bf16_rne(float f) {
    uint32_t u;
    memcpy(&u, &f, 4);
    if ((u & 0x7fffffffu) > 0x7f800000u) return (uint16_t)((u >> 16) | 0x40);
    u += 0x7fffu + ((u >> 16) & 1u);
    return (uint16_t)(u >> 16);
}

static Buf upload_f32(uzu_engine* e, const std::vector<float>& v) {
    Buf b = make_buf(e, std::max<size_t>(v.size() * 4, 16), UZU_BUFFER_DEVICE);
    cudaMemcpy((void*)b.ptr(), v.data(), v.size() * 4, cudaMemcpyHostToDevice);
    return b;
}

// `count` matrices [rows, cols] back to back, in the engine's storage type
static DenseMatrix upload_matrix(uzu_engine* e, const std::vector<float>& v, uint32_t rows, uint32_t cols, uint32_t count = 1) {
    if (v.size() != (size_t)rows * cols * count) throw std::runtime_error("internal: matrix assembly size mismatch");
    DenseMatrix m;
    m.rows = rows; m.cols = cols; m.count = count;
    m.bytes = v.size() * storage_size(e->store_dt);
    m.w = make_buf(e, std::max<size_t>(m.bytes, 16), UZU_BUFFER_DEVICE);
    if (e->store_dt == UZU_DT_F32) {
        cudaMemcpy((void*)m.w.ptr(), v.data(), m.bytes, cudaMemcpyHostToDevice);
    } else {
        std::vector<uint16_t> h(v.size());
        for (size_t i = 0; i < v.size(); ++i) h[i] = f32_to_bf16_rne(v[i]);
        cudaMemcpy((void*)m.w.ptr(), h.data(), m.bytes, cudaMemcpyHostToDevice);
    }
    return m;
}

static void append(std::vector<float>& dst, const HostTensor& t) { dst.insert(dst.end(), t.v.begin(), t.v.end()); }

static uint32_t cfg_u32(const Json& j, const char* key) {
    const Json& v = j.at(key);
    if (v.type != Json::Num || v.num < 0 || v.num != std::floor(v.num) || v.num > 4294967295.0) throw std::runtime_error(std::string("config: '") + key + "' must be a non-negative integer");
    return (uint32_t)v.num;
}

}  // namespace

static void load_parallel_block_model(uzu_engine* e, const Json& cfg, const std::string& dir) {
    if (e->opts.tp_size > 1) throw std::runtime_error("tensor parallelism is not built for the parallel-block family");
    e->parallel_block = true;
    e->store_dt = e->opts.storage_f32 ? UZU_DT_F32 : UZU_DT_BF16;
    const uint32_t W = e->model_dim = cfg_u32(cfg, "width");
    const uint32_t V = e->vocab = cfg_u32(cfg, "vocab");
    const Json& nc = cfg.at("norm");
    e->norm_eps = (float)nc.at("eps").number();
    e->norm_groups = cfg_u32(nc, "groups");
    if (e->norm_groups == 0 || W % e->norm_groups) throw std::runtime_error("config: width is not divisible into norm.groups parts");
    if (const Json* cap = cfg.get("logit_softcap")) {
        if (!cap->is_null()) { e->has_logit_soft_cap = true; e->logit_soft_cap = (float)cap->number(); }
    }
    ParameterLoader pl(dir + "/model.safetensors");
    e->pb_embed = upload_matrix(e, read_floats(pl, "embed", {V, W}).v, V, W);
    e->pb_head = upload_matrix(e, read_floats(pl, "head", {V, W}).v, V, W);
    e->pb_final_norm = upload_f32(e, read_floats(pl, "final.norm", {W}).v);
    uint64_t wbytes = e->pb_head.bytes, kvb = 0, stb = 0;
    uint32_t n_cache = 0, n_rec = 0;
    const auto& lcs = cfg.at("layers").arr;
    e->layers.resize(lcs.size());
    for (size_t i = 0; i < lcs.size(); ++i) {
        const Json& lc = lcs[i];
        Layer& L = e->layers[i];
        const std::string p = "l" + std::to_string(i) + ".";
        L.pre_mixer.present = true;
        L.pre_mixer.n = W;
        L.pre_mixer.cfg.epsilon = e->norm_eps;
        L.pre_mixer.scales = upload_f32(e, read_floats(pl, p + "norm1", {W}).v);
        const std::string type = lc.at("type").str;
        const Json& mc = lc.at("mixer");
        if (type == "general_delta") {
            L.kind = MixGeneralDelta;
            L.is_attention = false;
            GeneralDeltaLayer& G = L.gd;
            G.heads = cfg_u32(mc, "heads");
            G.dim = cfg_u32(mc, "dim");
            if (G.heads == 0 || G.dim == 0 || G.dim > 512) throw std::runtime_error(p + "mix: head size must be in 1..512");
            const uint32_t HD = G.heads * G.dim;
            auto it = pl.tensors.find(p + "mix.w1");
            if (it == pl.tensors.end() || it->second.shape.size() != 2) throw std::runtime_error("missing tensor '" + p + "mix.w1'");
            G.decay_rank = (uint32_t)it->second.shape[0];
            std::vector<float> in;
            for (const char* nm : {"r", "k", "v", "a", "g"}) append(in, read_floats(pl, p + "mix." + nm, {HD, W}));
            append(in, read_floats(pl, p + "mix.w1", {G.decay_rank, W}));
            G.in = upload_matrix(e, in, 5 * HD + G.decay_rank, W);
            G.decay_up = upload_matrix(e, read_floats(pl, p + "mix.w2", {HD, G.decay_rank}).v, HD, G.decay_rank);
            G.out = upload_matrix(e, read_floats(pl, p + "mix.o", {W, HD}).v, W, HD);
            G.rate_bias = upload_f32(e, read_floats(pl, p + "mix.a.b", {HD}).v);
            G.decay_bias = upload_f32(e, read_floats(pl, p + "mix.w0", {HD}).v);
            G.norm_weight = upload_f32(e, read_floats(pl, p + "mix.norm", {HD}).v);
            wbytes += G.in.bytes + G.decay_up.bytes + G.out.bytes;
            stb += 2ull * G.heads * G.dim * G.dim * 4;
            n_rec++;
        } else if (type == "latent_attention") {
            L.kind = MixLatentAttention;
            L.is_attention = true;
            LatentAttentionLayer& A = L.la;
            A.heads = cfg_u32(mc, "heads");
            A.dim = cfg_u32(mc, "dim");
            A.rot_dim = cfg_u32(mc, "rot_dim");
            A.vdim = cfg_u32(mc, "vdim");
            A.rank = cfg_u32(mc, "kv_rank");
            A.q_rank = cfg_u32(mc, "q_rank");
            A.scale = (float)mc.at("scale").number();
            if (A.heads == 0 || A.rank == 0 || A.rank > 512 || A.vdim == 0 || A.q_rank == 0) throw std::runtime_error(p + "mix: latent size must be in 1..512, heads / vdim / q_rank non-zero");
            if (A.rot_dim) {
                const Json& rot = mc.at("rot");
                RopeCfg rc;
                rc.kind = 3;
                rc.base = (float)rot.at("base").number();
                rc.head_dim = cfg_u32(rot, "dims");
                rc.max_sequence_length = 0xFFFFFFFFu;
                if (rc.head_dim % 2 || rc.head_dim > A.rot_dim) throw std::runtime_error(p + "mix: rot.dims must be even and at most rot_dim");
                const Json* sc = rot.get("scaling");
                if (sc && !sc->is_null()) {
                    rc.yarn = true;
                    rc.scaling_factor = (float)sc->at("factor").number();
                    rc.original_context_length = cfg_u32(*sc, "original");
                    rc.high = (float)sc->at("fast").number();
                    rc.low = (float)sc->at("slow").number();
                }
                int idx = -1;
                for (size_t r = 0; r < e->ropes.size(); ++r)
                    if (e->ropes[r] == rc) idx = (int)r;
                if (idx < 0) { e->ropes.push_back(rc); idx = (int)e->ropes.size() - 1; }
                A.rope_index = idx;
            }
            const uint32_t qd = A.dim + A.rot_dim;
            std::vector<float> in;
            append(in, read_floats(pl, p + "mix.dq", {A.q_rank, W}));
            append(in, read_floats(pl, p + "mix.dkv", {A.rank + A.rot_dim, W}));
            append(in, read_floats(pl, p + "mix.g", {A.heads * A.vdim, W}));
            A.in = upload_matrix(e, in, A.q_rank + A.rank + A.rot_dim + A.heads * A.vdim, W);
            A.kv_offset = A.q_rank;
            A.gate_offset = A.q_rank + A.rank + A.rot_dim;
            A.q_up = upload_matrix(e, read_floats(pl, p + "mix.uq", {A.heads * qd, A.q_rank}).v, A.heads * qd, A.q_rank);
            {   // per head the key up-projection [dim, rank] becomes [rank, dim]: q_abs = (W_uk^h)^T q^h as a linear with weight [out = rank, in = dim]
                HostTensor uk = read_floats(pl, p + "mix.uk", {A.heads * A.dim, A.rank});
                std::vector<float> t((size_t)A.heads * A.rank * std::max(A.dim, 1u));
                for (uint32_t h = 0; h < A.heads; ++h)
                    for (uint32_t d = 0; d < A.dim; ++d)
                        for (uint32_t r = 0; r < A.rank; ++r) t[((size_t)h * A.rank + r) * A.dim + d] = uk.v[((size_t)h * A.dim + d) * A.rank + r];
                t.resize((size_t)A.heads * A.rank * A.dim);
                if (A.dim) A.key_absorb = upload_matrix(e, t, A.rank, A.dim, A.heads);
            }
            A.value_up = upload_matrix(e, read_floats(pl, p + "mix.uv", {A.heads * A.vdim, A.rank}).v, A.vdim, A.rank, A.heads);
            A.out = upload_matrix(e, read_floats(pl, p + "mix.o", {W, A.heads * A.vdim}).v, W, A.heads * A.vdim);
            A.q_norm = upload_f32(e, read_floats(pl, p + "mix.dq.norm", {A.q_rank}).v);
            A.latent_norm = upload_f32(e, read_floats(pl, p + "mix.dkv.norm", {A.rank}).v);
            wbytes += A.in.bytes + A.q_up.bytes + A.key_absorb.bytes + A.value_up.bytes + A.out.bytes;
            kvb += (uint64_t)(A.rank + A.rot_dim) * storage_size(e->store_dt);
            n_cache++;
        } else {
            throw std::runtime_error("layer type '" + type + "' is not known to the parallel-block family");
        }
        GatedMlp& M = L.gmlp;
        const Json* ml = lc.get("mlp");
        if (ml && !ml->is_null()) {
            const std::string kind = ml->at("kind").str;
            if (kind == "dense") {
                M.kind = GatedMlp::Dense;
                M.f = cfg_u32(*ml, "ff");
                M.limit = (float)ml->at("limit").number();
                std::vector<float> gu;
                append(gu, read_floats(pl, p + "mlp.gate", {M.f, W}));
                append(gu, read_floats(pl, p + "mlp.up", {M.f, W}));
                M.gate_up = upload_matrix(e, gu, 2 * M.f, W);
                M.down = upload_matrix(e, read_floats(pl, p + "mlp.down", {W, M.f}).v, W, M.f);
                wbytes += M.gate_up.bytes + M.down.bytes;
            } else if (kind == "moe") {
                M.kind = GatedMlp::TableExperts;
                const Json& ex = ml->at("expert");
                const Json& ro = ml->at("router");
                M.f = cfg_u32(ex, "ff");
                M.limit = (float)ex.at("limit").number();
                M.experts = cfg_u32(ro, "experts");
                M.top = cfg_u32(ro, "top");
                if (M.experts == 0 || M.top == 0 || M.top > M.experts || M.experts > 8192 || (uint64_t)MAX_ROWS * M.top * 2 > 40000) throw std::runtime_error(p + "mlp: bad expert / top counts");
                std::vector<float> gu, dn;
                for (uint32_t x = 0; x < M.experts; ++x) {
                    const std::string q = p + "mlp.e" + std::to_string(x) + ".";
                    append(gu, read_floats(pl, q + "gate", {M.f, W}));
                    append(gu, read_floats(pl, q + "up", {M.f, W}));
                    append(dn, read_floats(pl, q + "down", {W, M.f}));
                }
                M.gate_up = upload_matrix(e, gu, 2 * M.f, W, M.experts);
                M.down = upload_matrix(e, dn, W, M.f, M.experts);
                const TensorInfo& tt = pl.validate(p + "mlp.table", {V, M.top}, "I32");
                M.table = make_buf(e, tt.end - tt.begin, UZU_BUFFER_MANAGED);
                pl.read_into(tt, uzu_buffer_cpu_ptr(M.table.b));
                check(uzu_buffer_make_resident(e->ctx, M.table.b));
                wbytes += (M.gate_up.bytes + M.down.bytes) / M.experts * M.top;
            } else {
                throw std::runtime_error("mlp kind '" + kind + "' is not known to the parallel-block family");
            }
        }
    }
    pl.assert_all_validated();
    e->info.model_dim = W;
    e->info.hidden_dim = 0;
    e->info.vocab_size = V;
    e->info.num_layers = (uint32_t)e->layers.size();
    e->info.num_attention_layers = n_cache;
    e->info.num_delta_net_layers = n_rec;
    e->info.weight_bytes_per_token = wbytes;
    e->info.kv_bytes_per_token_per_ctx = kvb;
    e->info.state_bytes_per_token = stb;
}

// Gamanex: sigmoid attention mixers (optionally reading an earlier layer's keys and values), relu^2 dense or routed silu-gated expert
// feed-forwards, two norms of the same input per layer, every sublayer's result times a per-channel scale and a sigmoid gate of its input.
// config.json: "width", "vocab", "norm": {"eps"}, "logit_scale", "layers": [{"type": "attention", "mixer": {"heads", "kv_heads", "dim",
// "vdim", "scale", "q_temp": {"coef", "every"}, "kv_from"}, "mlp": null | {"kind": "dense", "ff"} | {"kind": "moe", "expert": {"ff"},
// "router": {"experts", "top"}}}]. Tensors: l<i>.norm1/2, l<i>.mix.{q,k,v,o,q.norm,k.norm,r1,r2,pb}, l<i>.mlp.{up,down} or
// l<i>.mlp.{router,router.b,e<x>.{gate,up,down}}, l<i>.ls1/2, l<i>.rg1/2 (+ .b).
static void load_gamanex_model(uzu_engine* e, const Json& cfg, const std::string& dir) {
    if (e->opts.tp_size > 1) throw std::runtime_error("tensor parallelism is not built for the parallel-block families");
    e->parallel_block = true;
    e->store_dt = e->opts.storage_f32 ? UZU_DT_F32 : UZU_DT_BF16;
    const uint32_t W = e->model_dim = cfg_u32(cfg, "width");
    const uint32_t V = e->vocab = cfg_u32(cfg, "vocab");
    e->norm_eps = (float)cfg.at("norm").at("eps").number();
    e->norm_groups = 1;
    if (const Json* ls = cfg.get("logit_scale")) {
        if (!ls->is_null()) { e->has_logit_scale = true; e->logit_scale = (float)ls->number(); }
    }
    ParameterLoader pl(dir + "/model.safetensors");
    e->pb_embed = upload_matrix(e, read_floats(pl, "embed", {V, W}).v, V, W);
    e->pb_head = upload_matrix(e, read_floats(pl, "head", {V, W}).v, V, W);
    e->pb_final_norm = upload_f32(e, read_floats(pl, "final.norm", {W}).v);
    uint64_t wbytes = e->pb_head.bytes, kvb = 0;
    uint32_t n_cache = 0;
    const auto& lcs = cfg.at("layers").arr;
    e->layers.resize(lcs.size());
    // the gate matrix joins the sublayer's stacked projection (returns the rows it added); a checkpoint without the gate or without the
    // scale of a sublayer leaves that factor out
    auto sublayer_gate = [&](SublayerGate& g, std::vector<float>& stacked, uint32_t rows_before, const std::string& p, const char* scale, const char* gate) -> uint32_t {
        uint32_t added = 0;
        g.offset = rows_before;
        if (pl.tensors.count(p + gate)) {
            append(stacked, read_floats(pl, p + gate, {W, W}));
            g.bias = upload_f32(e, read_floats(pl, p + gate + ".b", {W}).v);
            added = W;
        }
        if (pl.tensors.count(p + scale)) g.scale = upload_f32(e, read_floats(pl, p + scale, {W}).v);
        g.present = g.bias.b || g.scale.b;
        return added;
    };
    for (size_t i = 0; i < lcs.size(); ++i) {
        const Json& lc = lcs[i];
        Layer& L = e->layers[i];
        const std::string p = "l" + std::to_string(i) + ".";
        L.pre_mixer.present = true;
        L.pre_mixer.n = W;
        L.pre_mixer.cfg.epsilon = e->norm_eps;
        L.pre_mixer.scales = upload_f32(e, read_floats(pl, p + "norm1", {W}).v);
        const std::string type = lc.at("type").str;
        if (type != "attention") throw std::runtime_error("layer type '" + type + "' is not known to the Gamanex family");
        const Json& mc = lc.at("mixer");
        L.kind = MixSigmoidAttention;
        L.is_attention = true;
        SigmoidAttentionLayer& A = L.sa;
        A.heads = cfg_u32(mc, "heads");
        A.kv_heads = cfg_u32(mc, "kv_heads");
        A.dim = cfg_u32(mc, "dim");
        A.vdim = cfg_u32(mc, "vdim");
        A.scale = (float)mc.at("scale").number();
        if (A.heads == 0 || A.kv_heads == 0 || A.heads % A.kv_heads || A.dim == 0 || A.vdim == 0 || A.dim > 512 || A.vdim > 512)
            throw std::runtime_error(p + "mix: kv_heads must divide heads, head sizes must be in 1..512");
        if (const Json* qt = mc.get("q_temp")) {
            if (!qt->is_null()) {
                A.temp_coef = (float)qt->at("coef").number();
                A.temp_every = cfg_u32(*qt, "every");
                if (A.temp_every == 0) throw std::runtime_error(p + "mix: q_temp.every must be positive");
            }
        }
        if (const Json* kf = mc.get("kv_from")) {
            if (!kf->is_null()) {
                A.kv_from = (int)cfg_u32(mc, "kv_from");
                if ((size_t)A.kv_from >= i) throw std::runtime_error(p + "mix: kv_from must name an earlier layer");
                const SigmoidAttentionLayer& src = e->layers[A.kv_from].sa;
                if (e->layers[A.kv_from].kind != MixSigmoidAttention || src.kv_from >= 0 || src.kv_heads != A.kv_heads || src.dim != A.dim || src.vdim != A.vdim)
                    throw std::runtime_error(p + "mix: kv_from must name a layer that keeps its own keys and values with the same head count and sizes");
            }
        }
        const uint32_t qn = A.heads * A.dim, kn = A.kv_heads * A.dim, vn = A.kv_heads * A.vdim;
        std::vector<float> in;
        append(in, read_floats(pl, p + "mix.q", {qn, W}));
        uint32_t rows = qn;
        A.q_norm = upload_f32(e, read_floats(pl, p + "mix.q.norm", {qn}).v);
        if (A.kv_from < 0) {
            append(in, read_floats(pl, p + "mix.k", {kn, W}));
            append(in, read_floats(pl, p + "mix.v", {vn, W}));
            A.k_norm = upload_f32(e, read_floats(pl, p + "mix.k.norm", {kn}).v);
            rows += kn + vn;
            kvb += (uint64_t)(kn + vn) * storage_size(e->store_dt);
            n_cache++;
        }
        rows += sublayer_gate(L.mix_gate, in, rows, p, "ls1", "rg1");
        A.in = upload_matrix(e, in, rows, W);
        A.out = upload_matrix(e, read_floats(pl, p + "mix.o", {W, A.heads * A.vdim}).v, W, A.heads * A.vdim);
        A.dist_r1 = upload_f32(e, read_floats(pl, p + "mix.r1", {A.heads}).v);
        A.dist_r2 = upload_f32(e, read_floats(pl, p + "mix.r2", {A.heads}).v);
        A.head_bias = upload_f32(e, read_floats(pl, p + "mix.pb", {A.heads}).v);
        wbytes += A.in.bytes + A.out.bytes;
        GatedMlp& M = L.gmlp;
        const Json* ml = lc.get("mlp");
        if (!ml || ml->is_null()) continue;
        L.pre_mlp.present = true;
        L.pre_mlp.n = W;
        L.pre_mlp.cfg.epsilon = e->norm_eps;
        L.pre_mlp.scales = upload_f32(e, read_floats(pl, p + "norm2", {W}).v);
        const std::string kind = ml->at("kind").str;
        if (kind == "dense") {
            M.kind = GatedMlp::Dense;
            M.unit = GatedMlp::ReluSquared;
            M.f = cfg_u32(*ml, "ff");
            if (M.f == 0) throw std::runtime_error(p + "mlp: ff must be positive");
            std::vector<float> up;
            append(up, read_floats(pl, p + "mlp.up", {M.f, W}));
            const uint32_t gate_rows = sublayer_gate(L.mlp_gate, up, M.f, p, "ls2", "rg2");
            M.gate_up = upload_matrix(e, up, M.f + gate_rows, W);
            M.down = upload_matrix(e, read_floats(pl, p + "mlp.down", {W, M.f}).v, W, M.f);
            wbytes += M.gate_up.bytes + M.down.bytes;
        } else if (kind == "moe") {
            M.kind = GatedMlp::RoutedExperts;
            M.unit = GatedMlp::SiluGlu;
            M.f = cfg_u32(ml->at("expert"), "ff");
            M.experts = cfg_u32(ml->at("router"), "experts");
            M.top = cfg_u32(ml->at("router"), "top");
            if (M.f == 0 || M.experts == 0 || M.top == 0 || M.top > M.experts || M.experts > 8192 || (uint64_t)MAX_ROWS * M.top * 2 > 40000)
                throw std::runtime_error(p + "mlp: bad expert / top counts");
            std::vector<float> ro, gu, dn;
            append(ro, read_floats(pl, p + "mlp.router", {M.experts, W}));
            const uint32_t gate_rows = sublayer_gate(L.mlp_gate, ro, M.experts, p, "ls2", "rg2");
            M.router = upload_matrix(e, ro, M.experts + gate_rows, W);
            M.router_bias = upload_f32(e, read_floats(pl, p + "mlp.router.b", {M.experts}).v);
            for (uint32_t x = 0; x < M.experts; ++x) {
                const std::string q = p + "mlp.e" + std::to_string(x) + ".";
                append(gu, read_floats(pl, q + "gate", {M.f, W}));
                append(gu, read_floats(pl, q + "up", {M.f, W}));
                append(dn, read_floats(pl, q + "down", {W, M.f}));
            }
            M.gate_up = upload_matrix(e, gu, 2 * M.f, W, M.experts);
            M.down = upload_matrix(e, dn, W, M.f, M.experts);
            wbytes += M.router.bytes + (M.gate_up.bytes + M.down.bytes) / M.experts * M.top;
        } else {
            throw std::runtime_error("mlp kind '" + kind + "' is not known to the Gamanex family");
        }
    }
    pl.assert_all_validated();
    e->info.model_dim = W;
    e->info.hidden_dim = 0;
    e->info.vocab_size = V;
    e->info.num_layers = (uint32_t)e->layers.size();
    e->info.num_attention_layers = n_cache;
    e->info.num_delta_net_layers = 0;
    e->info.weight_bytes_per_token = wbytes;
    e->info.kv_bytes_per_token_per_ctx = kvb;
    e->info.state_bytes_per_token = 0;
}

// Vugipel: sequential pre-norm layers (x <- x + mixer(n1(x)), then x <- x + ff(n2(x))) whose norm weights are stored as distances from
// one; mixers: minGRU, or window attention and retention side by side (both read the same normed input, their outputs are summed with
// fixed shares); feed-forward: routed silu-gated experts whose sigmoid router weight multiplies the expert's INPUT, or none.
// config.json: "width", "vocab", "norm": {"eps"}, "layers": [{"type": "mingru", "mixer": {"width"}} | {"type": "parallel", "mixer":
// {"left": {"heads", "kv_heads", "dim", "vdim", "scale", "softcap", "rot": {"base", "dims"}, "mask": {"size", "keep_first"}}, "left_scale",
// "right": {"heads", "dim", "vdim", "decay": [..]}, "right_scale"}}, each with "mlp": null | {"kind": "moe", "expert": {"ff"}, "router":
// {"experts", "top"}}]. Tensors: l<i>.norm1/2, l<i>.mix.{z,z.b,x,x.b,g,o} | l<i>.mix.left.{q,k,v,o (+ .b), q.norm, k.norm, temp},
// l<i>.mix.right.{q,k,v,g,o}; l<i>.mlp.{router, e<x>.{gate,up,down}}.
static void load_vugipel_model(uzu_engine* e, const Json& cfg, const std::string& dir) {
    if (e->opts.tp_size > 1) throw std::runtime_error("tensor parallelism is not built for the parallel-block families");
    e->parallel_block = true;
    e->store_dt = e->opts.storage_f32 ? UZU_DT_F32 : UZU_DT_BF16;
    const uint32_t W = e->model_dim = cfg_u32(cfg, "width");
    const uint32_t V = e->vocab = cfg_u32(cfg, "vocab");
    e->norm_eps = (float)cfg.at("norm").at("eps").number();
    e->norm_groups = 1;
    ParameterLoader pl(dir + "/model.safetensors");
    // a norm weight w stands for the factor 1 + w (formed once, in f32)
    auto offset_norm = [&](const std::string& name) {
        HostTensor t = read_floats(pl, name, {W});
        for (float& v : t.v) v = 1.0f + v;
        return upload_f32(e, t.v);
    };
    auto rope = [&](float base, uint32_t dims) {
        RopeCfg rc;
        rc.kind = 3;
        rc.base = base;
        rc.head_dim = dims;
        rc.max_sequence_length = 0xFFFFFFFFu;
        for (size_t r = 0; r < e->ropes.size(); ++r)
            if (e->ropes[r] == rc) return (int)r;
        e->ropes.push_back(rc);
        return (int)e->ropes.size() - 1;
    };
    e->pb_embed = upload_matrix(e, read_floats(pl, "embed", {V, W}).v, V, W);
    e->pb_head = upload_matrix(e, read_floats(pl, "head", {V, W}).v, V, W);
    e->pb_final_norm = offset_norm("final.norm");
    uint64_t wbytes = e->pb_head.bytes, kvb = 0, stb = 0;
    uint32_t n_cache = 0, n_rec = 0;
    const auto& lcs = cfg.at("layers").arr;
    e->layers.resize(lcs.size());
    for (size_t i = 0; i < lcs.size(); ++i) {
        const Json& lc = lcs[i];
        Layer& L = e->layers[i];
        const std::string p = "l" + std::to_string(i) + ".";
        L.sequential = true;
        L.pre_mixer.present = true;
        L.pre_mixer.n = W;
        L.pre_mixer.cfg.epsilon = e->norm_eps;
        L.pre_mixer.scales = offset_norm(p + "norm1");
        const std::string type = lc.at("type").str;
        const Json& mc = lc.at("mixer");
        if (type == "mingru") {
            L.kind = MixMinGru;
            L.is_attention = false;
            MinGruLayer& G = L.mg;
            G.width = cfg_u32(mc, "width");
            if (G.width == 0) throw std::runtime_error(p + "mix: width must be positive");
            std::vector<float> in, bias;
            append(in, read_floats(pl, p + "mix.z", {G.width, W}));
            append(in, read_floats(pl, p + "mix.x", {G.width, W}));
            append(in, read_floats(pl, p + "mix.g", {G.width, W}));
            append(bias, read_floats(pl, p + "mix.z.b", {G.width}));
            append(bias, read_floats(pl, p + "mix.x.b", {G.width}));
            bias.resize((size_t)3 * G.width, 0.0f);
            G.in = upload_matrix(e, in, 3 * G.width, W);
            G.in_bias = upload_f32(e, bias);
            G.out = upload_matrix(e, read_floats(pl, p + "mix.o", {W, G.width}).v, W, G.width);
            wbytes += G.in.bytes + G.out.bytes;
            stb += 2ull * G.width * 4;
            n_rec++;
        } else if (type == "parallel") {
            L.kind = MixSideBySide;
            L.is_attention = true;
            WindowAttentionLayer& A = L.wa;
            RetentionLayer& R = L.rt;
            const Json& lj = mc.at("left");
            const Json& rj = mc.at("right");
            A.heads = cfg_u32(lj, "heads");
            A.kv_heads = cfg_u32(lj, "kv_heads");
            A.dim = cfg_u32(lj, "dim");
            A.vdim = cfg_u32(lj, "vdim");
            A.scale = (float)lj.at("scale").number();
            A.share = (float)mc.at("left_scale").number();
            if (const Json* sc = lj.get("softcap")) { if (!sc->is_null()) A.softcap = (float)sc->number(); }
            if (const Json* mk = lj.get("mask")) {
                if (!mk->is_null()) { A.window = cfg_u32(*mk, "size"); A.keep_first = cfg_u32(*mk, "keep_first"); }
            }
            if (A.heads == 0 || A.kv_heads == 0 || A.heads % A.kv_heads || A.dim == 0 || A.vdim == 0 || A.dim > 512 || A.vdim > 512)
                throw std::runtime_error(p + "mix.left: kv_heads must divide heads, head sizes must be in 1..512");
            if (A.softcap < 0.0f) throw std::runtime_error(p + "mix.left: softcap must not be negative");
            if (const Json* rot = lj.get("rot")) {
                if (!rot->is_null()) {
                    const float base = (float)rot->at("base").number();
                    const uint32_t dims = cfg_u32(*rot, "dims");
                    if (dims % 2 || dims > A.dim || A.vdim % 2) throw std::runtime_error(p + "mix.left: rot.dims must be even and at most dim, vdim must be even");
                    if (dims) A.rope_index = rope(base, dims);
                    A.value_rope_index = rope(base, A.vdim);         // values turn over all their channels, with frequencies of their own
                }
            }
            R.heads = cfg_u32(rj, "heads");
            R.dim = cfg_u32(rj, "dim");
            R.vdim = cfg_u32(rj, "vdim");
            R.share = (float)mc.at("right_scale").number();
            if (R.heads == 0 || R.dim == 0 || R.dim > 1024 || R.vdim == 0) throw std::runtime_error(p + "mix.right: heads / vdim must be positive, dim in 1..1024");
            {
                const auto& dj = rj.at("decay").arr;
                if (dj.size() != R.heads) throw std::runtime_error(p + "mix.right: one decay per head is expected");
                std::vector<float> d;
                for (const Json& x : dj) d.push_back((float)x.number());
                R.decay = upload_f32(e, d);
            }
            const uint32_t lq = A.heads * A.dim, lk = A.kv_heads * A.dim, lv = A.kv_heads * A.vdim, rq = R.heads * R.dim, rv = R.heads * R.vdim;
            const std::string l = p + "mix.left.", r = p + "mix.right.";
            std::vector<float> in, bias;
            append(in, read_floats(pl, l + "q", {lq, W}));
            append(in, read_floats(pl, l + "k", {lk, W}));
            append(in, read_floats(pl, l + "v", {lv, W}));
            append(in, read_floats(pl, r + "q", {rq, W}));
            append(in, read_floats(pl, r + "k", {rq, W}));
            append(in, read_floats(pl, r + "v", {rv, W}));
            append(in, read_floats(pl, r + "g", {rv, W}));
            append(bias, read_floats(pl, l + "q.b", {lq}));
            append(bias, read_floats(pl, l + "k.b", {lk}));
            append(bias, read_floats(pl, l + "v.b", {lv}));
            A.q_offset = 0; A.k_offset = lq; A.v_offset = lq + lk;
            R.q_offset = lq + lk + lv; R.k_offset = R.q_offset + rq; R.v_offset = R.k_offset + rq; R.gate_offset = R.v_offset + rv;
            const uint32_t rows = R.gate_offset + rv;
            bias.resize(rows, 0.0f);
            L.side_in = upload_matrix(e, in, rows, W);
            L.side_in_bias = upload_f32(e, bias);
            A.q_norm = upload_f32(e, read_floats(pl, l + "q.norm", {A.dim}).v);
            A.k_norm = upload_f32(e, read_floats(pl, l + "k.norm", {A.dim}).v);
            A.head_temp = upload_f32(e, read_floats(pl, l + "temp", {A.heads}).v);
            A.out = upload_matrix(e, read_floats(pl, l + "o", {W, A.heads * A.vdim}).v, W, A.heads * A.vdim);
            {
                HostTensor ob = read_floats(pl, l + "o.b", {W});
                for (float& v : ob.v) v *= A.share;
                A.out_bias = upload_f32(e, ob.v);
            }
            R.out = upload_matrix(e, read_floats(pl, r + "o", {W, rv}).v, W, rv);
            wbytes += L.side_in.bytes + A.out.bytes + R.out.bytes;
            kvb += (uint64_t)(lk + lv) * storage_size(e->store_dt);
            stb += 2ull * R.heads * R.dim * R.vdim * 4;
            n_cache++;
            n_rec++;
        } else {
            throw std::runtime_error("layer type '" + type + "' is not known to the Vugipel family");
        }
        GatedMlp& M = L.gmlp;
        const Json* ml = lc.get("mlp");
        if (!ml || ml->is_null()) {
            if (pl.tensors.count(p + "norm2")) read_floats(pl, p + "norm2", {W});       // a norm without a sublayer: checked, not used
            continue;
        }
        L.pre_mlp.present = true;
        L.pre_mlp.n = W;
        L.pre_mlp.cfg.epsilon = e->norm_eps;
        L.pre_mlp.scales = offset_norm(p + "norm2");
        const std::string kind = ml->at("kind").str;
        if (kind != "moe") throw std::runtime_error("mlp kind '" + kind + "' is not known to the Vugipel family");
        M.kind = GatedMlp::RoutedExperts;
        M.unit = GatedMlp::SiluGlu;
        M.sigmoid_weights = true;
        M.weight_on_input = true;
        M.f = cfg_u32(ml->at("expert"), "ff");
        M.experts = cfg_u32(ml->at("router"), "experts");
        M.top = cfg_u32(ml->at("router"), "top");
        if (M.f == 0 || M.experts == 0 || M.top == 0 || M.top > M.experts || M.experts > 8192 || (uint64_t)MAX_ROWS * M.top * 2 > 40000)
            throw std::runtime_error(p + "mlp: bad expert / top counts");
        std::vector<float> gu, dn;
        M.router = upload_matrix(e, read_floats(pl, p + "mlp.router", {M.experts, W}).v, M.experts, W);
        for (uint32_t x = 0; x < M.experts; ++x) {
            const std::string q = p + "mlp.e" + std::to_string(x) + ".";
            append(gu, read_floats(pl, q + "gate", {M.f, W}));
            append(gu, read_floats(pl, q + "up", {M.f, W}));
            append(dn, read_floats(pl, q + "down", {W, M.f}));
        }
        M.gate_up = upload_matrix(e, gu, 2 * M.f, W, M.experts);
        M.down = upload_matrix(e, dn, W, M.f, M.experts);
        wbytes += M.router.bytes + (M.gate_up.bytes + M.down.bytes) / M.experts * M.top;
    }
    pl.assert_all_validated();
    e->info.model_dim = W;
    e->info.hidden_dim = 0;
    e->info.vocab_size = V;
    e->info.num_layers = (uint32_t)e->layers.size();
    e->info.num_attention_layers = n_cache;
    e->info.num_delta_net_layers = n_rec;
    e->info.weight_bytes_per_token = wbytes;
    e->info.kv_bytes_per_token_per_ctx = kvb;
    e->info.state_bytes_per_token = stb;
}

// Vakesun: sequential sandwich layers, x <- x + m * post(sublayer(pre(x))) with Dynamic Tanh norms (tanh(alpha x) w + b) before AND after
// every sublayer and a fixed factor m on every addition; a per-layer token input after the feed-forward (a gelu unit of the residual,
// gated by a row of a second embedding table, projected, RMS-normed and added); scaled input embedding, readout with the embedding table.
// Mixers: softmax attention with grouped key / value heads, per-head q / k RMS norms and a half-split rotation with YaRN-blended
// frequencies ("attention": the window-attention kernels without a window); a matrix memory with exponential gates ("mlstm"); latent
// attention without positions, with a sliding window, a sink term per head, a sigmoid gate per head and optionally another layer's
// latent cache ("latent_attention"). Feed-forward: relu^2.
// config.json: "width", "vocab", "norm": {"eps"}, "residual_mult", "embedding": {"scale"}, "token_side": {"dim"}, "layers": [{"type",
// "mixer": {...}, "mlp": null | {"kind": "dense", "ff"}}]. Tensors: embed, side.embed, final.norm (+ .b, .alpha), l<i>.norm1 / norm1b /
// norm2 / norm2b (+ .b, .alpha), l<i>.mix.*, l<i>.mlp.{up,down}, l<i>.side.{gate,proj,norm}.
static void load_vakesun_model(uzu_engine* e, const Json& cfg, const std::string& dir) {
    if (e->opts.tp_size > 1) throw std::runtime_error("tensor parallelism is not built for the parallel-block families");
    e->parallel_block = true;
    e->store_dt = e->opts.storage_f32 ? UZU_DT_F32 : UZU_DT_BF16;
    const uint32_t W = e->model_dim = cfg_u32(cfg, "width");
    const uint32_t V = e->vocab = cfg_u32(cfg, "vocab");
    e->norm_eps = (float)cfg.at("norm").at("eps").number();
    e->norm_groups = 1;
    const float mult = (float)cfg.at("residual_mult").number();
    if (const Json* em = cfg.get("embedding")) {
        if (!em->is_null()) e->input_scale = (float)em->at("scale").number();
    }
    uint32_t side_dim = 0;
    if (const Json* ts = cfg.get("token_side")) {
        if (!ts->is_null()) side_dim = cfg_u32(*ts, "dim");
    }
    ParameterLoader pl(dir + "/model.safetensors");
    auto dyt = [&](const std::string& name) {
        Norm n;
        n.present = true;
        n.kind = 1;
        n.n = W;
        n.cfg.epsilon = e->norm_eps;
        n.scales = upload_f32(e, read_floats(pl, name, {W}).v);
        n.bias = upload_f32(e, read_floats(pl, name + ".b", {W}).v);
        n.alpha = read_floats(pl, name + ".alpha", {}).v[0];
        return n;
    };
    const auto& lcs = cfg.at("layers").arr;
    e->pb_embed = upload_matrix(e, read_floats(pl, "embed", {V, W}).v, V, W);
    e->pb_head = e->pb_embed;        // the readout multiplies with the embedding table itself (without the input scale)
    if (side_dim) e->pb_side_embed = upload_matrix(e, read_floats(pl, "side.embed", {V, (uint64_t)lcs.size() * side_dim}).v, V, (uint32_t)lcs.size() * side_dim);
    e->pb_out_norm = dyt("final.norm");
    uint64_t wbytes = e->pb_head.bytes, kvb = 0, stb = 0;
    uint32_t n_cache = 0, n_rec = 0;
    e->layers.resize(lcs.size());
    for (size_t i = 0; i < lcs.size(); ++i) {
        const Json& lc = lcs[i];
        Layer& L = e->layers[i];
        const std::string p = "l" + std::to_string(i) + ".";
        L.sequential = true;
        L.sandwich = true;
        L.residual_mult = mult;
        L.pre_mixer = dyt(p + "norm1");
        L.post_mixer = dyt(p + "norm1b");
        const std::string type = lc.at("type").str;
        const Json& mc = lc.at("mixer");
        if (type == "attention") {
            L.kind = MixWindowAttention;
            L.is_attention = true;
            WindowAttentionLayer& A = L.wa;
            A.heads = cfg_u32(mc, "heads");
            A.kv_heads = cfg_u32(mc, "kv_heads");
            A.dim = cfg_u32(mc, "dim");
            A.vdim = cfg_u32(mc, "vdim");
            A.scale = (float)mc.at("scale").number();
            if (A.heads == 0 || A.kv_heads == 0 || A.heads % A.kv_heads || A.dim == 0 || A.vdim == 0 || A.dim > 512 || A.vdim > 512)
                throw std::runtime_error(p + "mix: kv_heads must divide heads, head sizes must be in 1..512");
            if (const Json* rot = mc.get("rot")) {
                if (!rot->is_null() && cfg_u32(*rot, "dims")) {
                    RopeCfg rc;
                    rc.kind = 3;                 // a table row holds the cos / sin of the pairs, whatever channels a pair is made of
                    rc.base = (float)rot->at("base").number();
                    rc.head_dim = cfg_u32(*rot, "dims");
                    rc.max_sequence_length = 0xFFFFFFFFu;
                    if (rc.head_dim % 2 || rc.head_dim > A.dim) throw std::runtime_error(p + "mix: rot.dims must be even and at most dim");
                    const Json* sc = rot->get("scaling");
                    if (sc && !sc->is_null()) {
                        rc.yarn = true;
                        rc.scaling_factor = (float)sc->at("factor").number();
                        rc.original_context_length = cfg_u32(*sc, "original");
                        rc.high = (float)sc->at("fast").number();
                        rc.low = (float)sc->at("slow").number();
                    }
                    int idx = -1;
                    for (size_t r = 0; r < e->ropes.size(); ++r)
                        if (e->ropes[r] == rc) idx = (int)r;
                    if (idx < 0) { e->ropes.push_back(rc); idx = (int)e->ropes.size() - 1; }
                    A.rope_index = idx;
                    A.rot_halves = true;
                }
            }
            const uint32_t qn = A.heads * A.dim, kn = A.kv_heads * A.dim, vn = A.kv_heads * A.vdim;
            std::vector<float> in;
            append(in, read_floats(pl, p + "mix.q", {qn, W}));
            append(in, read_floats(pl, p + "mix.k", {kn, W}));
            append(in, read_floats(pl, p + "mix.v", {vn, W}));
            A.q_offset = 0; A.k_offset = qn; A.v_offset = qn + kn;
            L.side_in = upload_matrix(e, in, qn + kn + vn, W);
            A.q_norm = upload_f32(e, read_floats(pl, p + "mix.q.norm", {A.dim}).v);
            A.k_norm = upload_f32(e, read_floats(pl, p + "mix.k.norm", {A.dim}).v);
            A.out = upload_matrix(e, read_floats(pl, p + "mix.o", {W, A.heads * A.vdim}).v, W, A.heads * A.vdim);
            wbytes += L.side_in.bytes + A.out.bytes;
            kvb += (uint64_t)(kn + vn) * storage_size(e->store_dt);
            n_cache++;
        } else if (type == "mlstm") {
            L.kind = MixMlstm;
            L.is_attention = false;
            MlstmLayer& M = L.ml;
            M.heads = cfg_u32(mc, "heads");
            M.dim = cfg_u32(mc, "dim");
            M.vdim = cfg_u32(mc, "vdim");
            M.gate_cap = (float)mc.at("gate_cap").number();
            if (M.heads == 0 || M.dim == 0 || M.dim > 1024 || M.vdim == 0 || M.gate_cap < 0.0f) throw std::runtime_error(p + "mix: heads / vdim must be positive, dim in 1..1024, gate_cap not negative");
            const uint32_t qn = M.heads * M.dim, vn = M.heads * M.vdim;
            std::vector<float> in, bias;
            append(in, read_floats(pl, p + "mix.q", {qn, W}));
            append(in, read_floats(pl, p + "mix.k", {qn, W}));
            append(in, read_floats(pl, p + "mix.v", {vn, W}));
            append(in, read_floats(pl, p + "mix.g", {vn, W}));
            append(in, read_floats(pl, p + "mix.i", {M.heads, W}));
            append(in, read_floats(pl, p + "mix.f", {M.heads, W}));
            M.q_offset = 0; M.k_offset = qn; M.v_offset = 2 * qn; M.gate_offset = 2 * qn + vn; M.i_offset = 2 * qn + 2 * vn; M.f_offset = M.i_offset + M.heads;
            bias.assign(M.i_offset, 0.0f);
            append(bias, read_floats(pl, p + "mix.i.b", {M.heads}));
            append(bias, read_floats(pl, p + "mix.f.b", {M.heads}));
            M.in = upload_matrix(e, in, M.f_offset + M.heads, W);
            M.in_bias = upload_f32(e, bias);
            M.norm_weight = upload_f32(e, read_floats(pl, p + "mix.norm", {vn}).v);
            M.out = upload_matrix(e, read_floats(pl, p + "mix.o", {W, vn}).v, W, vn);
            wbytes += M.in.bytes + M.out.bytes;
            stb += 2ull * M.heads * M.dim * (M.vdim + 1) * 4;
            n_rec++;
        } else if (type == "latent_attention") {
            L.kind = MixLatentAttention;
            L.is_attention = true;
            LatentAttentionLayer& A = L.la;
            A.heads = cfg_u32(mc, "heads");
            A.dim = cfg_u32(mc, "dim");
            A.vdim = cfg_u32(mc, "vdim");
            A.rank = cfg_u32(mc, "kv_rank");
            A.q_rank = cfg_u32(mc, "q_rank");
            A.scale = (float)mc.at("scale").number();
            A.gate_per_head = true;
            if (A.heads == 0 || A.dim == 0 || A.rank == 0 || A.rank > 512 || A.vdim == 0 || A.q_rank == 0) throw std::runtime_error(p + "mix: latent size must be in 1..512, heads / dim / vdim / q_rank non-zero");
            if (const Json* mk = mc.get("mask")) {
                if (!mk->is_null()) A.window = cfg_u32(*mk, "size");
            }
            if (const Json* kf = mc.get("kv_from")) {
                if (!kf->is_null()) {
                    A.kv_from = (int)cfg_u32(mc, "kv_from");
                    if ((size_t)A.kv_from >= i) throw std::runtime_error(p + "mix: kv_from must name an earlier layer");
                    const Layer& src = e->layers[A.kv_from];
                    if (src.kind != MixLatentAttention || src.la.kv_from >= 0 || src.la.rank != A.rank || src.la.rot_dim != 0)
                        throw std::runtime_error(p + "mix: kv_from must name a latent-attention layer that keeps its own latents of the same size");
                }
            }
            std::vector<float> in;
            append(in, read_floats(pl, p + "mix.dq", {A.q_rank, W}));
            uint32_t rows = A.q_rank;
            if (A.kv_from < 0) {
                A.kv_offset = rows;
                append(in, read_floats(pl, p + "mix.dkv", {A.rank, W}));
                rows += A.rank;
                A.latent_norm = upload_f32(e, read_floats(pl, p + "mix.dkv.norm", {A.rank}).v);
                n_cache++;
            }
            // bytes a decode step reads from the latent cache (the lender's rows, also for a borrower): the window's rows, or the whole context
            if (A.window) stb += (uint64_t)A.window * A.rank * storage_size(e->store_dt);
            else kvb += (uint64_t)A.rank * storage_size(e->store_dt);
            A.gate_offset = rows;
            append(in, read_floats(pl, p + "mix.g", {A.heads, W}));
            rows += A.heads;
            A.in = upload_matrix(e, in, rows, W);
            A.q_up = upload_matrix(e, read_floats(pl, p + "mix.uq", {A.heads * A.dim, A.q_rank}).v, A.heads * A.dim, A.q_rank);
            {   // per head the key up-projection [dim, rank] becomes [rank, dim] (the absorbed form: the query meets the cached latent itself)
                HostTensor uk = read_floats(pl, p + "mix.uk", {A.heads * A.dim, A.rank});
                std::vector<float> t((size_t)A.heads * A.rank * A.dim);
                for (uint32_t h = 0; h < A.heads; ++h)
                    for (uint32_t d = 0; d < A.dim; ++d)
                        for (uint32_t r = 0; r < A.rank; ++r) t[((size_t)h * A.rank + r) * A.dim + d] = uk.v[((size_t)h * A.dim + d) * A.rank + r];
                A.key_absorb = upload_matrix(e, t, A.rank, A.dim, A.heads);
            }
            {
                HostTensor uv = read_floats(pl, p + "mix.uv", {A.heads * A.vdim, A.rank});
                A.value_up = upload_matrix(e, uv.v, A.vdim, A.rank, A.heads);
                // long prompt passes in bf16 expand the latents of their window into keys and values (one product on the tensor-memory kernel)
                // and run the tensor-pipe softmax attention on them: a second copy of the two up-projections, stacked
                if (e->store_dt == UZU_DT_BF16 && A.rank % 64 == 0 && A.dim % 16 == 0 && A.vdim % 16 == 0 && A.dim <= 128 && A.vdim <= 128) {
                    std::vector<float> kv = read_floats(pl, p + "mix.uk", {A.heads * A.dim, A.rank}).v;
                    kv.insert(kv.end(), uv.v.begin(), uv.v.end());
                    A.kv_up = upload_matrix(e, kv, A.heads * (A.dim + A.vdim), A.rank);
                }
            }
            A.out = upload_matrix(e, read_floats(pl, p + "mix.o", {W, A.heads * A.vdim}).v, W, A.heads * A.vdim);
            A.q_norm = upload_f32(e, read_floats(pl, p + "mix.dq.norm", {A.q_rank}).v);
            A.sink = upload_f32(e, read_floats(pl, p + "mix.sink", {A.heads}).v);
            wbytes += A.in.bytes + A.q_up.bytes + A.key_absorb.bytes + A.value_up.bytes + A.out.bytes;
        } else {
            throw std::runtime_error("layer type '" + type + "' is not known to the Vakesun family");
        }
        if (side_dim) {
            TokenSide& T = L.side;
            T.present = true;
            T.dim = side_dim;
            T.column = (uint32_t)i * side_dim;
            T.gate = upload_matrix(e, read_floats(pl, p + "side.gate", {side_dim, W}).v, side_dim, W);
            T.proj = upload_matrix(e, read_floats(pl, p + "side.proj", {W, side_dim}).v, W, side_dim);
            T.norm = upload_f32(e, read_floats(pl, p + "side.norm", {W}).v);
            wbytes += T.gate.bytes + T.proj.bytes + (uint64_t)side_dim * storage_size(e->store_dt);
        }
        GatedMlp& M = L.gmlp;
        const Json* ml = lc.get("mlp");
        if (!ml || ml->is_null()) continue;
        L.pre_mlp = dyt(p + "norm2");
        L.post_mlp = dyt(p + "norm2b");
        const std::string kind = ml->at("kind").str;
        if (kind != "dense") throw std::runtime_error("mlp kind '" + kind + "' is not known to the Vakesun family");
        M.kind = GatedMlp::Dense;
        M.unit = GatedMlp::ReluSquared;
        M.f = cfg_u32(*ml, "ff");
        if (M.f == 0) throw std::runtime_error(p + "mlp: ff must be positive");
        M.gate_up = upload_matrix(e, read_floats(pl, p + "mlp.up", {M.f, W}).v, M.f, W);
        M.down = upload_matrix(e, read_floats(pl, p + "mlp.down", {W, M.f}).v, W, M.f);
        wbytes += M.gate_up.bytes + M.down.bytes;
    }
    pl.assert_all_validated();
    e->info.model_dim = W;
    e->info.hidden_dim = 0;
    e->info.vocab_size = V;
    e->info.num_layers = (uint32_t)e->layers.size();
    e->info.num_attention_layers = n_cache;
    e->info.num_delta_net_layers = n_rec;
    e->info.weight_bytes_per_token = wbytes;
    e->info.kv_bytes_per_token_per_ctx = kvb;
    e->info.state_bytes_per_token = stb;
}

constexpr uint32_t kPromptChunks = 8;  // most key chunks of a row tile of a sigmoid-attention prompt pass
constexpr uint32_t kSplitRows = 256;   // query rows x key splits of one latent-attention launch that leaves partial softmax states

// scratch of the family: f32 row blocks sized by the widest layer
static void create_parallel_block_scratch(uzu_engine* e) {
    if (!e->parallel_block) return;
    const uint32_t W = e->model_dim;
    uint32_t proj = 1, lat = 1, wide = 1, query = 1, mixed = 1, gated = 1, gu = 1, act = 1, top = 1, experts = 1, partial = 1, kmax = e->model_dim;
    uint32_t proj2 = 1, tickets = 1, prompt_partial = 0, factor_heads = 0, expand_cols = 0, expand_rows = 0;
    bool second_norm = false, sandwich = false;
    for (const Layer& L : e->layers) {
        second_norm = second_norm || L.pre_mlp.present;
        sandwich = sandwich || L.sandwich;
        if (L.side.present) { lat = std::max(lat, L.side.dim); kmax = std::max(kmax, L.side.dim); }
        if (L.kind == MixSigmoidAttention) {
            const SigmoidAttentionLayer& A = L.sa;
            proj = std::max(proj, A.in.rows);
            query = std::max(query, A.heads * A.dim);
            mixed = std::max(mixed, A.heads * A.vdim);
            partial = std::max(partial, A.heads * A.vdim);
            if (e->store_dt == UZU_DT_BF16) prompt_partial = std::max(prompt_partial, A.heads * A.vdim);    // chunked tensor-pipe prompt passes
            tickets = std::max(tickets, A.heads);
            kmax = std::max(kmax, A.heads * A.vdim);
        } else if (L.kind == MixMlstm) {
            proj = std::max(proj, L.ml.in.rows);
            wide = std::max(wide, L.ml.heads * L.ml.vdim);
            gated = std::max(gated, L.ml.heads * L.ml.vdim);
            kmax = std::max(kmax, L.ml.heads * L.ml.vdim);
            factor_heads = std::max(factor_heads, L.ml.heads);
        } else if (L.kind == MixMinGru) {
            proj = std::max(proj, L.mg.in.rows);
            gated = std::max(gated, L.mg.width);
            kmax = std::max(kmax, L.mg.width);
        } else if (L.has_window_attention() || L.has_retention()) {
            proj = std::max(proj, L.side_in.rows);
            if (L.has_window_attention()) {
                const WindowAttentionLayer& A = L.wa;
                query = std::max(query, A.heads * A.dim);
                mixed = std::max(mixed, A.heads * A.vdim);
                partial = std::max(partial, A.heads * (A.vdim + 2));
                tickets = std::max(tickets, A.heads);
                kmax = std::max(kmax, A.heads * A.vdim);
            }
            if (L.has_retention()) {
                wide = std::max(wide, L.rt.heads * L.rt.vdim);
                gated = std::max(gated, L.rt.heads * L.rt.vdim);
                kmax = std::max(kmax, L.rt.heads * L.rt.vdim);
            }
        } else if (L.kind == MixGeneralDelta) {
            const uint32_t HD = L.gd.heads * L.gd.dim;
            proj = std::max(proj, L.gd.in.rows);
            lat = std::max(lat, L.gd.decay_rank);
            wide = std::max(wide, HD);
            mixed = std::max(mixed, HD);
            gated = std::max(gated, HD);
            kmax = std::max({kmax, HD, L.gd.decay_rank});
        } else {
            const LatentAttentionLayer& A = L.la;
            proj = std::max(proj, A.in.rows);
            lat = std::max(lat, A.q_rank);
            wide = std::max(wide, A.heads * (A.dim + A.rot_dim));
            query = std::max(query, A.heads * (A.rank + A.rot_dim));
            mixed = std::max(mixed, A.heads * A.rank);
            gated = std::max(gated, A.heads * A.vdim);
            partial = std::max(partial, A.heads * (A.rank + 2));
            kmax = std::max({kmax, A.q_rank, A.heads * A.vdim});
            if (A.kv_up.w.b) {      // rows a pass may expand: its own, the window before them (from a tile's edge), or the whole context without a window
                expand_cols = std::max(expand_cols, A.kv_up.rows);
                expand_rows = std::max(expand_rows, MAX_ROWS + (A.window ? A.window + 64 : e->max_context));
            }
        }
        if (L.gmlp.kind == GatedMlp::RoutedExperts) proj2 = std::max(proj2, L.gmlp.router.rows);
        if (L.gmlp.unit == GatedMlp::ReluSquared) proj2 = std::max(proj2, L.gmlp.gate_up.rows);
        if (L.gmlp.kind != GatedMlp::None) {
            gu = std::max(gu, 2 * L.gmlp.f);
            act = std::max(act, L.gmlp.f);
            kmax = std::max(kmax, L.gmlp.f);
            top = std::max(top, L.gmlp.top);
            experts = std::max(experts, L.gmlp.experts);
        }
    }
    auto dev = [&](size_t bytes) { return make_buf(e, std::max<size_t>(bytes, 256), UZU_BUFFER_DEVICE); };
    const size_t R = MAX_ROWS;
    auto& P = e->pb;
    P.resid = dev(R * W * 4);
    P.normed = dev(R * W * 4);
    if (second_norm) P.normed2 = dev(R * W * 4);
    if (sandwich) P.sub_out = dev(R * W * 4);
    if (factor_heads) P.token_factors = dev(4 * R * factor_heads * 4);
    if (expand_cols) {
        P.expand_rows = std::min(expand_rows, 16384u);      // longer ranges take the kernel that reads the latents directly
        P.expand_f32 = dev((size_t)P.expand_rows * expand_cols * 4);
        P.expand_keys = dev((size_t)P.expand_rows * expand_cols * 2);
        P.expand_values = dev((size_t)P.expand_rows * expand_cols * 2);
    }
    P.proj2 = dev(R * proj2 * 4);
    P.pair_weight = dev(R * top * 4);
    P.pair_weight_compact = dev(R * top * 4);
    P.route_scratch = dev(R * top * 2);
    P.attn_tickets = dev((size_t)kSplitRows * tickets * 4);
    cudaMemset((void*)P.attn_tickets.ptr(), 0, (size_t)kSplitRows * tickets * 4);
    P.operand_bf16 = dev(R * kmax * 2);     // bf16 copy of a prompt pass's activation rows for the tensor-memory products
    P.proj = dev(R * proj * 4);
    P.lat = dev(R * lat * 4);
    P.wide = dev(R * wide * 4);
    P.lat_wide = dev(R * wide * 4);     // unit keys of a prompt pass (generalized delta rule)
    P.query = dev(R * query * 4);
    P.attn_partial = dev(std::max((size_t)kSplitRows * partial, (size_t)prompt_partial * kPromptChunks * R) * 4);
    P.mixed = dev(R * mixed * 4);
    P.gated_mix = dev(R * std::max(gated, mixed) * 4);
    P.gate_up = dev(R * top * gu * 4);
    P.act = dev(R * top * act * 4);
    P.pair_out = dev(R * top * W * 4);
    P.group_offsets = dev((size_t)(experts + 1) * 4);
    P.rows_map = dev(R * top * 4);
    P.pair_pos = dev(R * top * 4);
    P.normed_rows = dev((size_t)e->logits_rows * W * 4);
    P.logits_f32 = dev((size_t)e->logits_rows * e->vocab * 4);
}

static uzu_dense_linear_args dense_args(const uzu_engine* e, const DenseMatrix& m, uint64_t a, uint32_t rows, uint64_t d) {
    uzu_dense_linear_args x{};
    x.a = a; x.w = m.w.ptr(); x.d = d;
    x.m = rows; x.n = m.rows; x.k = m.cols; x.lda = m.cols; x.ldd = m.rows; x.batch = 1;
    x.weights_dt = e->store_dt; x.scale = 1.0f;
    x.workspace = e->pb.operand_bf16.ptr();
    return x;
}

static void encode_dense(uzu_engine* e, uzu_command_buffer* cmd, const DenseMatrix& m, uint64_t a, uint32_t lda, uint32_t rows, uint64_t d) {
    uzu_dense_linear_args x = dense_args(e, m, a, rows, d);
    x.lda = lda;
    uzu_dense_linear_encode(cmd, &x);
}

// A sandwich layer's short pass: the output projection's epilogue norms the product, adds it into the residual stream and norms the
// updated stream for the next reader (both norms are Dynamic Tanh, elementwise), instead of a launch of its own after the projection.
static void sublayer_epilogue(uzu_engine* e, uzu_dense_linear_args& x) {
    auto& P = e->pb;
    if (!P.fused_post) return;
    x.d = P.resid.ptr(); x.accumulate = 0;
    x.post_weight = P.fused_post->scales.ptr(); x.post_bias = P.fused_post->bias.ptr(); x.post_alpha = P.fused_post->alpha; x.post_mult = P.fused_mult;
    if (P.fused_reader) {
        x.next_out = P.normed.ptr(); x.next_weight = P.fused_reader->scales.ptr(); x.next_bias = P.fused_reader->bias.ptr(); x.next_alpha = P.fused_reader->alpha;
    }
}

// x += A . W^T: the sublayers' output projections add straight into the residual stream. With a sublayer gate the product is first
// multiplied by scale[c] * sigmoid(logits[row, c] + bias[c]); the logits are columns [offset, offset + width) of a [rows, gate_ld] block.
static void encode_into_residual(uzu_engine* e, uzu_command_buffer* cmd, const DenseMatrix& w, uint64_t a, uint32_t lda, uint32_t rows,
                                 const SublayerGate* g = nullptr, uint64_t gate_block = 0, uint32_t gate_ld = 0, uint32_t a_op = 0) {
    // (a sandwich layer's sublayer leaves its result in a scratch block: it goes through a norm of its own before it is added)
    uzu_dense_linear_args x = dense_args(e, w, a, rows, e->pb.redirect ? e->pb.sub_out.ptr() : e->pb.resid.ptr());
    x.lda = lda; x.accumulate = e->pb.redirect ? 0 : 1; x.a_op = a_op;
    sublayer_epilogue(e, x);
    if (g && g->present) {
        if (g->bias.b) { x.gate = gate_block + (uint64_t)g->offset * 4; x.gate_ld = gate_ld; x.gate_bias = g->bias.ptr(); }
        if (g->scale.b) x.col_scale = g->scale.ptr();
    }
    uzu_dense_linear_encode(cmd, &x);
}

// h [m, W] -> sigmoid attention over the layer's own cache or the cache of the layer it borrows from; the output projection adds into the
// residual stream through the sublayer gate
static void encode_sigmoid_attention(uzu_engine* e, uzu_command_buffer* cmd, const Layer& L, LayerState& own, const PassCtx& pc) {
    const SigmoidAttentionLayer& A = L.sa;
    auto& P = e->pb;
    LayerState& C = A.kv_from >= 0 ? e->state[A.kv_from] : own;      // the lender ran earlier in this pass: its rows of the pass are in place
    const uint32_t m = pc.m, ld = A.in.rows, qn = A.heads * A.dim, kn = A.kv_heads * A.dim, vn = A.kv_heads * A.vdim;
    const uint64_t dyn = pc.dynamic ? e->decode_state.ptr() : 0;
    encode_dense(e, cmd, A.in, P.normed.ptr(), e->model_dim, m, P.proj.ptr());            // [query | key | value | gate logits]
    uzu_sigmoid_attention_prepare_args pa{};
    pa.q = P.proj.ptr(); pa.q_scales = A.q_norm.ptr(); pa.query = P.query.ptr();
    if (A.kv_from < 0) {
        pa.k = P.proj.ptr() + (uint64_t)qn * 4; pa.v = P.proj.ptr() + (uint64_t)(qn + kn) * 4; pa.k_scales = A.k_norm.ptr();
        pa.keys = C.keys; pa.values = C.values;
    }
    pa.dynamic_position = dyn;
    pa.rows = m; pa.q_n = qn; pa.k_n = kn; pa.v_n = vn; pa.q_stride = pa.k_stride = pa.v_stride = ld;
    pa.prefix = C.length; pa.cache_dt = e->store_dt; pa.temp_every = A.temp_every; pa.temp_coef = A.temp_coef; pa.epsilon = e->norm_eps;
    uzu_sigmoid_attention_prepare_encode(cmd, &pa);
    uzu_sigmoid_attention_args aa{};
    aa.query = P.query.ptr(); aa.keys = C.keys; aa.values = C.values; aa.out = P.mixed.ptr(); aa.dynamic_position = dyn;
    aa.dist_r1 = A.dist_r1.ptr(); aa.dist_r2 = A.dist_r2.ptr(); aa.head_bias = A.head_bias.ptr();
    aa.rows = m; aa.heads = A.heads; aa.kv_heads = A.kv_heads; aa.dim = A.dim; aa.vdim = A.vdim; aa.prefix = C.length; aa.cache_dt = e->store_dt;
    aa.scale = A.scale;
    {   // few query rows (decode, short portions): cut the keys (in tiles of 16) so that about eight small CTAs per SM run and a warp walks
        // its keys in one to four rounds (the captured step sizes the cut for the largest context its graph serves)
        const uint32_t bound = pc.dynamic ? attention_bucket(C.length + m) : C.length + m;
        const uint32_t tiles = (bound + 15) / 16;
        const uint32_t want = std::max(1u, 8u * (uint32_t)e->ctx->sm_count / std::max(1u, m * A.heads));
        aa.splits = std::min({tiles, want, kSplitRows / std::max(1u, m), 128u});
        aa.partials = P.attn_partial.ptr(); aa.tickets = P.attn_tickets.ptr();
        if (aa.splits < 2 || m > kSplitRows) aa.splits = 1;
        // long passes on the tensor pipe: at most kPromptChunks chunks of at least 4 key tiles per row tile (the partial tiles fit the scratch)
        if (!pc.dynamic && m >= 64) aa.chunk_tiles = std::max(4u, ((C.length + m + 63) / 64 + kPromptChunks - 1) / kPromptChunks);
    }
    uzu_sigmoid_attention_encode(cmd, &aa);
    encode_into_residual(e, cmd, A.out, P.mixed.ptr(), A.heads * A.vdim, m, &L.mix_gate, P.proj.ptr(), ld);
}

// h [m, W] -> minGRU: one stacked projection [gate logits | candidate | output gate] with its biases, the scan over the pass with the
// state carried in S, and the output projection that adds into the residual stream
static void encode_min_gru(uzu_engine* e, uzu_command_buffer* cmd, const Layer& L, LayerState& S, const PassCtx& pc) {
    const MinGruLayer& G = L.mg;
    auto& P = e->pb;
    const uint32_t m = pc.m, ld = G.in.rows;
    {
        uzu_dense_linear_args x = dense_args(e, G.in, P.normed.ptr(), m, P.proj.ptr());
        x.lda = e->model_dim; x.bias = G.in_bias.ptr();
        uzu_dense_linear_encode(cmd, &x);
    }
    uzu_min_gru_args ga{};
    ga.z_logit = P.proj.ptr(); ga.u = P.proj.ptr() + (uint64_t)G.width * 4; ga.gate = P.proj.ptr() + (uint64_t)2 * G.width * 4;
    ga.state = S.ssm_state.ptr(); ga.out = P.gated_mix.ptr();
    ga.rows = m; ga.n = G.width; ga.z_stride = ga.u_stride = ga.gate_stride = ld; ga.out_stride = G.width;
    uzu_min_gru_encode(cmd, &ga);
    encode_into_residual(e, cmd, G.out, P.gated_mix.ptr(), G.width, m);
}

// Window attention and / or retention reading the same normed input through ONE stacked projection; each output projection adds its share
// into the residual stream.
static void encode_side_by_side(uzu_engine* e, uzu_command_buffer* cmd, const Layer& L, LayerState& S, const PassCtx& pc) {
    auto& P = e->pb;
    const uint32_t m = pc.m, ld = L.side_in.rows;
    const uint64_t dyn = pc.dynamic ? e->decode_state.ptr() : 0;
    {
        uzu_dense_linear_args x = dense_args(e, L.side_in, P.normed.ptr(), m, P.proj.ptr());
        x.lda = e->model_dim;
        if (L.side_in_bias.b) x.bias = L.side_in_bias.ptr();
        uzu_dense_linear_encode(cmd, &x);
    }
    if (L.has_window_attention()) {
        const WindowAttentionLayer& A = L.wa;
        const uint64_t vcos = A.value_rope_index >= 0 ? e->rope_cos[A.value_rope_index].ptr() : 0, vsin = A.value_rope_index >= 0 ? e->rope_sin[A.value_rope_index].ptr() : 0;
        const uint32_t v_pairs = A.value_rope_index >= 0 ? A.vdim / 2 : 0;
        uzu_window_attention_prepare_args pa{};
        pa.q = P.proj.ptr() + (uint64_t)A.q_offset * 4; pa.k = P.proj.ptr() + (uint64_t)A.k_offset * 4; pa.v = P.proj.ptr() + (uint64_t)A.v_offset * 4;
        pa.q_scales = A.q_norm.ptr(); pa.k_scales = A.k_norm.ptr(); pa.query = P.query.ptr(); pa.keys = S.keys; pa.values = S.values;
        if (A.rope_index >= 0) {
            pa.cosines = e->rope_cos[A.rope_index].ptr(); pa.sines = e->rope_sin[A.rope_index].ptr();
            pa.rot_pairs = e->ropes[A.rope_index].head_dim / 2;
        }
        pa.v_cosines = vcos; pa.v_sines = vsin; pa.v_pairs = v_pairs; pa.dynamic_position = dyn;
        pa.rows = m; pa.heads = A.heads; pa.kv_heads = A.kv_heads; pa.dim = A.dim; pa.vdim = A.vdim;
        pa.q_stride = pa.k_stride = pa.v_stride = ld; pa.prefix = S.length; pa.cache_dt = e->store_dt; pa.epsilon = e->norm_eps;
        pa.rot_halves = A.rot_halves ? 1 : 0;
        uzu_window_attention_prepare_encode(cmd, &pa);
        uzu_window_attention_args aa{};
        aa.query = P.query.ptr(); aa.keys = S.keys; aa.values = S.values; aa.out = P.mixed.ptr(); aa.dynamic_position = dyn;
        aa.head_temp = A.head_temp.ptr(); aa.v_cosines = vcos; aa.v_sines = vsin; aa.v_pairs = v_pairs;
        aa.rows = m; aa.heads = A.heads; aa.kv_heads = A.kv_heads; aa.dim = A.dim; aa.vdim = A.vdim; aa.prefix = S.length; aa.cache_dt = e->store_dt;
        aa.window = A.window; aa.keep_first = A.keep_first; aa.scale = A.scale; aa.softcap = A.softcap;
        {   // few query rows: cut the visible keys (in tiles of 16) so that about eight small CTAs per SM run (the captured step sizes the
            // cut for the largest context its graph serves; a window bounds it)
            uint32_t bound = pc.dynamic ? attention_bucket(S.length + m) : S.length + m;
            if (A.window) bound = std::min(bound, A.window + A.keep_first);
            const uint32_t tiles = (bound + 15) / 16;
            const uint32_t want = std::max(1u, 8u * (uint32_t)e->ctx->sm_count / std::max(1u, m * A.heads));
            aa.splits = std::min({tiles, want, kSplitRows / std::max(1u, m), 128u});
            aa.partials = P.attn_partial.ptr(); aa.tickets = P.attn_tickets.ptr();
            if (aa.splits < 2 || m > kSplitRows) aa.splits = 1;
        }
        uzu_window_attention_encode(cmd, &aa);
        uzu_dense_linear_args x = dense_args(e, A.out, P.mixed.ptr(), m, P.redirect ? P.sub_out.ptr() : P.resid.ptr());
        x.lda = A.heads * A.vdim; x.accumulate = P.redirect ? 0 : 1; x.scale = A.share;
        if (A.out_bias.b) x.bias = A.out_bias.ptr();
        sublayer_epilogue(e, x);
        uzu_dense_linear_encode(cmd, &x);
    }
    if (L.has_retention()) {
        const RetentionLayer& R = L.rt;
        const uint32_t rv = R.heads * R.vdim;
        uzu_retention_args ra{};
        ra.q = P.proj.ptr() + (uint64_t)R.q_offset * 4; ra.k = P.proj.ptr() + (uint64_t)R.k_offset * 4; ra.v = P.proj.ptr() + (uint64_t)R.v_offset * 4;
        ra.decay = R.decay.ptr(); ra.state = S.ssm_state.ptr(); ra.out = P.wide.ptr();
        ra.rows = m; ra.heads = R.heads; ra.dim = R.dim; ra.vdim = R.vdim; ra.q_stride = ra.k_stride = ra.v_stride = ld; ra.out_stride = rv;
        ra.key_scale = 1.0f / sqrtf((float)R.dim);
        uzu_retention_encode(cmd, &ra);
        uzu_head_norm_gate_args na{};
        na.x = P.wide.ptr(); na.gate = P.proj.ptr() + (uint64_t)R.gate_offset * 4; na.out = P.gated_mix.ptr();
        na.rows = m; na.heads = R.heads; na.dim = R.vdim; na.x_stride = rv; na.gate_stride = ld; na.out_stride = rv; na.normalize = 1;
        na.epsilon = e->norm_eps; na.gate_op = 1;
        uzu_head_norm_gate_encode(cmd, &na);
        uzu_dense_linear_args x = dense_args(e, R.out, P.gated_mix.ptr(), m, P.redirect ? P.sub_out.ptr() : P.resid.ptr());
        x.lda = rv; x.accumulate = (P.redirect && !L.has_window_attention()) ? 0 : 1; x.scale = R.share;       // the second of two mixers adds to the first
        if (!L.has_window_attention()) sublayer_epilogue(e, x);
        uzu_dense_linear_encode(cmd, &x);
    }
}

// h [m, W] -> the mixer's output is added to the residual stream
static void encode_general_delta(uzu_engine* e, uzu_command_buffer* cmd, const Layer& L, LayerState& S, const PassCtx& pc) {
    const GeneralDeltaLayer& G = L.gd;
    auto& P = e->pb;
    const uint32_t m = pc.m, HD = G.heads * G.dim, ld = G.in.rows;
    encode_dense(e, cmd, G.in, P.normed.ptr(), e->model_dim, m, P.proj.ptr());            // [r | k | v | rate | gate | decay latent]
    {   // decay logits [m, HD] = W_up tanh(decay latent): the tanh is applied as the latent is read
        uzu_dense_linear_args x = dense_args(e, G.decay_up, P.proj.ptr() + (uint64_t)5 * HD * 4, m, P.wide.ptr());
        x.lda = ld; x.a_op = 1;
        uzu_dense_linear_encode(cmd, &x);
    }
    uzu_general_delta_args ga{};
    ga.r = P.proj.ptr(); ga.k = P.proj.ptr() + (uint64_t)HD * 4; ga.v = P.proj.ptr() + (uint64_t)2 * HD * 4;
    ga.rate_logit = P.proj.ptr() + (uint64_t)3 * HD * 4; ga.decay_logit = P.wide.ptr();
    ga.rate_bias = G.rate_bias.ptr(); ga.decay_bias = G.decay_bias.ptr();
    ga.state = S.ssm_state.ptr(); ga.out = P.mixed.ptr(); ga.unit = P.lat_wide.ptr();
    ga.r_stride = ga.k_stride = ga.v_stride = ga.rate_stride = ld; ga.decay_stride = HD;
    ga.rows = m; ga.heads = G.heads; ga.dim = G.dim;
    uzu_general_delta_encode(cmd, &ga);
    uzu_head_norm_gate_args na{};
    na.x = P.mixed.ptr(); na.scales = G.norm_weight.ptr(); na.gate = P.proj.ptr() + (uint64_t)4 * HD * 4; na.out = P.gated_mix.ptr();
    na.rows = m; na.heads = G.heads; na.dim = G.dim; na.x_stride = HD; na.gate_stride = ld; na.out_stride = HD; na.normalize = 1;
    na.epsilon = e->norm_eps;
    uzu_head_norm_gate_encode(cmd, &na);
    encode_into_residual(e, cmd, G.out, P.gated_mix.ptr(), HD, m);
}

static void encode_latent_attention(uzu_engine* e, uzu_command_buffer* cmd, const Layer& L, LayerState& own, const PassCtx& pc) {
    const LatentAttentionLayer& A = L.la;
    auto& P = e->pb;
    LayerState& S = A.kv_from >= 0 ? e->state[A.kv_from] : own;      // a lender ran earlier in this pass: its rows of the pass are in place
    const uint32_t m = pc.m, ld = A.in.rows, qd = A.dim + A.rot_dim, width = A.rank + A.rot_dim;
    const uint64_t dyn = pc.dynamic ? e->decode_state.ptr() : 0;
    encode_dense(e, cmd, A.in, P.normed.ptr(), e->model_dim, m, P.proj.ptr());            // [query latent | kv latent | rotated key | gate]; a borrower has no kv part
    const bool q_norm_in_prepare = A.rot_dim == 0;      // without a rotated query part the prepare launch does not wait for q: it norms the query latent too
    if (!q_norm_in_prepare) {
        uzu_group_rms_norm_args qn{};
        qn.input = P.proj.ptr(); qn.scales = A.q_norm.ptr(); qn.output = P.lat.ptr();
        qn.rows = m; qn.n = A.q_rank; qn.groups = 1; qn.in_stride = ld; qn.out_stride = A.q_rank; qn.epsilon = e->norm_eps;
        uzu_group_rms_norm_encode(cmd, &qn);
        encode_dense(e, cmd, A.q_up, P.lat.ptr(), A.q_rank, m, P.wide.ptr());              // q [m, heads, dim + rot_dim]
    }
    uzu_latent_prepare_args pa{};
    pa.kv = A.kv_from < 0 ? P.proj.ptr() + (uint64_t)A.kv_offset * 4 : 0; pa.q = A.rot_dim ? P.wide.ptr() : 0; pa.query = P.query.ptr(); pa.cache = S.keys;
    pa.latent_scales = A.latent_norm.ptr();
    if (A.rope_index >= 0) {
        pa.cosines = e->rope_cos[A.rope_index].ptr(); pa.sines = e->rope_sin[A.rope_index].ptr();
        pa.rot_pairs = e->ropes[A.rope_index].head_dim / 2;
    }
    pa.dynamic_position = dyn;
    pa.rows = m; pa.heads = A.heads; pa.dim = A.dim; pa.rot_dim = A.rot_dim; pa.rank = A.rank; pa.kv_stride = ld; pa.q_stride = A.heads * qd;
    pa.prefix = S.length; pa.cache_dt = e->store_dt; pa.epsilon = e->norm_eps;
    if (q_norm_in_prepare) { pa.q_latent = P.proj.ptr(); pa.q_latent_scales = A.q_norm.ptr(); pa.q_latent_out = P.lat.ptr(); pa.q_rank = A.q_rank; pa.q_latent_stride = ld; }
    if (pa.kv || pa.q || pa.q_latent) uzu_latent_prepare_encode(cmd, &pa);
    if (q_norm_in_prepare) encode_dense(e, cmd, A.q_up, P.lat.ptr(), A.q_rank, m, P.wide.ptr());      // q [m, heads, dim]
    // Long prompt passes over a bf16 cache: the latents of the visible range become keys and values per head again (one product on the
    // tensor-memory kernel, A = the cache rows as they are), stored as bf16, and the tensor-pipe softmax attention runs on them with the
    // sink and the head gate; its output is the heads' weighted value sums, so no value projection follows. The range starts at a key
    // tile's edge (64) at or before the first visible row; the temporary rows are addressed by their absolute position.
    if (A.kv_up.w.b && !pc.dynamic && m >= 64 && A.rot_dim == 0 && A.gate_per_head) {
        const uint32_t first_seen = A.window && S.length + 1 > A.window ? S.length + 1 - A.window : 0u;
        const uint32_t lo = first_seen / 64 * 64, rows = S.length + m - lo;
        const uint32_t kn = A.heads * A.dim, vn = A.heads * A.vdim;
        if (rows >= 128 && rows <= P.expand_rows && (S.keys & 15) == 0) {
            uzu_dense_linear_args x = dense_args(e, A.kv_up, S.keys + (uint64_t)lo * A.rank * 2, rows, P.expand_f32.ptr());
            x.a_bf16 = 1; x.lda = A.rank;
            uzu_dense_linear_encode(cmd, &x);
            uzu_rows_to_bf16_encode(cmd, P.expand_f32.ptr(), kn + vn, P.expand_keys.ptr(), rows, kn);
            uzu_rows_to_bf16_encode(cmd, P.expand_f32.ptr() + (uint64_t)kn * 4, kn + vn, P.expand_values.ptr(), rows, vn);
            uzu_window_attention_args wa{};
            wa.query = P.wide.ptr(); wa.out = P.gated_mix.ptr();
            wa.keys = P.expand_keys.ptr() - (uint64_t)lo * kn * 2; wa.values = P.expand_values.ptr() - (uint64_t)lo * vn * 2;     // row j of the cache is row j - lo here
            wa.rows = m; wa.heads = A.heads; wa.kv_heads = A.heads; wa.dim = A.dim; wa.vdim = A.vdim; wa.prefix = S.length; wa.cache_dt = UZU_DT_BF16;
            wa.window = A.window; wa.scale = A.scale; wa.splits = 1;
            wa.sinks = A.sink.ptr(); wa.head_gate = P.proj.ptr() + (uint64_t)A.gate_offset * 4; wa.head_gate_stride = ld;
            uzu_window_attention_encode(cmd, &wa);
            encode_into_residual(e, cmd, A.out, P.gated_mix.ptr(), vn, m);
            return;
        }
    }
    if (A.dim) {   // absorbed key projection, one z per head: query[:, h, 0:rank] = q[:, h, 0:dim] . (W_uk^h as [rank, dim])^T
        uzu_dense_linear_args x = dense_args(e, A.key_absorb, P.wide.ptr(), m, P.query.ptr());
        x.lda = A.heads * qd; x.ldd = A.heads * width; x.batch = A.heads;
        x.a_z_stride = qd; x.w_z_stride = A.key_absorb.stride(); x.d_z_stride = width;
        uzu_dense_linear_encode(cmd, &x);
    } else {
        cmd->record_error(UZU_ERROR_UNSUPPORTED, "latent attention without an unrotated key part is not built");
    }
    uzu_latent_attention_args aa{};
    aa.query = P.query.ptr(); aa.cache = S.keys; aa.out = P.mixed.ptr(); aa.dynamic_position = dyn;
    aa.rows = m; aa.heads = A.heads; aa.rank = A.rank; aa.rot_dim = A.rot_dim; aa.prefix = S.length; aa.cache_dt = e->store_dt; aa.scale = A.scale;
    aa.window = A.window; aa.sinks = A.sink.ptr();
    if (A.gate_per_head) { aa.head_gate = P.proj.ptr() + (uint64_t)A.gate_offset * 4; aa.head_gate_stride = ld; }
    {   // few query rows (decode, short portions): cut the keys so that about two CTAs per SM run. A captured step sizes the cut for the
        // largest context its graph serves (the graph is captured again when the context outgrows that); a window bounds it.
        uint32_t bound = pc.dynamic ? attention_bucket(S.length + m) : S.length + m;
        if (A.window) bound = std::min(bound, A.window + 31);
        const uint32_t tiles = (bound + 31) / 32, groups = (A.heads + 7) / 8;
        const uint32_t want = std::max(1u, 2u * (uint32_t)e->ctx->sm_count / std::max(1u, m * groups));
        aa.splits = std::min({tiles, want, kSplitRows / std::max(1u, m), 64u});
        aa.partials = P.attn_partial.ptr();
        if (aa.splits < 2 || m > kSplitRows) aa.splits = 1;
    }
    uzu_latent_attention_encode(cmd, &aa);
    {   // value projection per head, times the output gate: o[:, h, :] = (sum_j p_j c_j) . (W_uv^h)^T * sigmoid(gate[:, h, :])
        uzu_dense_linear_args x = dense_args(e, A.value_up, P.mixed.ptr(), m, P.gated_mix.ptr());
        x.lda = A.heads * A.rank; x.ldd = A.heads * A.vdim; x.batch = A.heads;
        x.a_z_stride = A.rank; x.w_z_stride = A.value_up.stride(); x.d_z_stride = A.vdim;
        if (!A.gate_per_head) { x.gate = P.proj.ptr() + (uint64_t)A.gate_offset * 4; x.gate_ld = ld; }     // (a gate per head is applied by the attention kernel)
        uzu_dense_linear_encode(cmd, &x);
    }
    encode_into_residual(e, cmd, A.out, P.gated_mix.ptr(), A.heads * A.vdim, m);
}

// h [m, W] -> matrix memory with exponential gates: one stacked projection [q | k | v | output gate | input-gate logit | forget-gate logit]
// with the two gate biases, the gates' scan (running maximum carried in the state), the gated linear recurrence with its normaliser
// column, then per head: division by max(|n . q|, exp(-m)) + 1e-6, unit RMS, weight, sigmoid gate; the output projection follows.
static void encode_mlstm(uzu_engine* e, uzu_command_buffer* cmd, const Layer& L, LayerState& S, const PassCtx& pc) {
    const MlstmLayer& M = L.ml;
    auto& P = e->pb;
    const uint32_t m = pc.m, ld = M.in.rows, vn = M.heads * M.vdim;
    {
        uzu_dense_linear_args x = dense_args(e, M.in, P.normed.ptr(), m, P.proj.ptr());
        x.lda = e->model_dim; x.bias = M.in_bias.ptr();
        uzu_dense_linear_encode(cmd, &x);
    }
    const uint64_t block = (uint64_t)MAX_ROWS * M.heads * 4;
    const uint64_t decay = P.token_factors.ptr(), gain = decay + block, floor = gain + block, nq = floor + block;
    const uint64_t matrix_floats = (uint64_t)M.heads * M.dim * (M.vdim + 1);
    uzu_exp_gates_args ga{};
    ga.i_pre = P.proj.ptr() + (uint64_t)M.i_offset * 4; ga.f_pre = P.proj.ptr() + (uint64_t)M.f_offset * 4;
    ga.state = S.ssm_state.ptr() + matrix_floats * 4;
    ga.token_decay = decay; ga.token_gain = gain; ga.floor = floor;
    ga.rows = m; ga.heads = M.heads; ga.i_stride = ga.f_stride = ld; ga.cap = M.gate_cap;
    uzu_exp_gates_encode(cmd, &ga);
    uzu_retention_args ra{};
    ra.q = P.proj.ptr() + (uint64_t)M.q_offset * 4; ra.k = P.proj.ptr() + (uint64_t)M.k_offset * 4; ra.v = P.proj.ptr() + (uint64_t)M.v_offset * 4;
    ra.state = S.ssm_state.ptr(); ra.out = P.wide.ptr();
    ra.rows = m; ra.heads = M.heads; ra.dim = M.dim; ra.vdim = M.vdim; ra.q_stride = ra.k_stride = ra.v_stride = ld; ra.out_stride = vn;
    ra.key_scale = 1.0f; ra.query_scale = 1.0f / sqrtf((float)M.dim);
    ra.token_decay = decay; ra.token_gain = gain; ra.norm_out = nq;
    uzu_retention_encode(cmd, &ra);
    uzu_head_norm_gate_args na{};
    na.x = P.wide.ptr(); na.scales = M.norm_weight.ptr(); na.gate = P.proj.ptr() + (uint64_t)M.gate_offset * 4; na.out = P.gated_mix.ptr();
    na.rows = m; na.heads = M.heads; na.dim = M.vdim; na.x_stride = vn; na.gate_stride = ld; na.out_stride = vn; na.normalize = 1;
    na.epsilon = e->norm_eps; na.gate_op = 0;
    na.denom = nq; na.denom_floor = floor; na.denom_epsilon = 1e-6f;
    uzu_head_norm_gate_encode(cmd, &na);
    encode_into_residual(e, cmd, M.out, P.gated_mix.ptr(), vn, m);
}

// h [m, W] -> the feed-forward output is added to the residual stream. Passes of at most 8 rows (decode) form gate and up in one launch
// that stores the gated unit; longer passes run the stacked [gate | up] product and the unit as two kernels.
// `h` is the sublayer's normed input [m, W]. Units: the clamped gated unit, silu(g) * u, or relu(u)^2 (no gate rows; the square is
// applied as the down projection reads its operand). A sublayer gate's logits come out of the first product of the sublayer (extra rows
// of the up matrix or of the router) and are applied where the result enters the residual stream.
static void encode_gated_mlp(uzu_engine* e, uzu_command_buffer* cmd, const Layer& L, const PassCtx& pc, uint64_t h) {
    const GatedMlp& M = L.gmlp;
    auto& P = e->pb;
    const uint32_t m = pc.m, W = e->model_dim;
    constexpr float kGateSlope = 1.702f;
    const bool paired = m <= 8;
    auto gate_up_args = [&]() {
        uzu_dense_linear_args up = dense_args(e, M.gate_up, h, m, paired ? P.act.ptr() : P.gate_up.ptr());
        up.lda = W;
        if (M.weight_on_input) up.row_scale = P.pair_weight_compact.ptr();      // expert(w h): the first product is linear in its input
        if (paired) { up.n = M.f; up.ldd = M.f; up.pair_rows = M.f; up.glu_limit = M.limit; up.glu_alpha = kGateSlope; up.glu_kind = M.unit == GatedMlp::SiluGlu ? 1 : 0; }
        return up;
    };
    auto unit = [&](uint32_t rows) {
        if (M.unit == GatedMlp::SiluGlu) uzu_silu_glu_encode(cmd, P.gate_up.ptr(), P.act.ptr(), rows, M.f);
        else uzu_clamped_glu_encode(cmd, P.gate_up.ptr(), P.act.ptr(), rows, M.f, M.limit, kGateSlope);
    };
    if (M.kind == GatedMlp::Dense && M.unit == GatedMlp::ReluSquared) {
        const uint32_t ld = M.gate_up.rows;                                       // [up | gate logits]
        encode_dense(e, cmd, M.gate_up, h, W, m, P.proj2.ptr());
        encode_into_residual(e, cmd, M.down, P.proj2.ptr(), ld, m, &L.mlp_gate, P.proj2.ptr(), ld, 2);
        return;
    }
    if (M.kind == GatedMlp::Dense) {
        uzu_dense_linear_args up = gate_up_args();
        uzu_dense_linear_encode(cmd, &up);
        if (!paired) unit(m);
        encode_into_residual(e, cmd, M.down, P.act.ptr(), M.f, m);
        return;
    }
    // routed experts: expert-sorted (token, slot) pairs, grouped products over the pairs, weighted combine per token
    if (M.kind == GatedMlp::RoutedExperts) {
        encode_dense(e, cmd, M.router, h, W, m, P.proj2.ptr());                   // [router logits | gate logits]
        uzu_topk_route_args ra{};
        ra.logits = P.proj2.ptr(); ra.bias = M.router_bias.ptr(); ra.group_offsets = P.group_offsets.ptr(); ra.rows_map = P.rows_map.ptr();
        ra.pair_pos = P.pair_pos.ptr(); ra.pair_weight = P.pair_weight.ptr(); ra.rows = m; ra.top = M.top; ra.experts = M.experts;
        ra.logits_stride = M.router.rows;
        ra.weight_kind = M.sigmoid_weights ? 1 : 0;
        ra.scratch = P.route_scratch.ptr();
        if (M.weight_on_input) ra.compact_weight = P.pair_weight_compact.ptr();
        if (!M.router_bias.b) ra.bias = 0;
        uzu_topk_route_encode(cmd, &ra);
    } else {
        uzu_table_route_args ra{};
        ra.token_ids = e->token_ids.ptr(); ra.table = M.table.ptr(); ra.group_offsets = P.group_offsets.ptr(); ra.rows_map = P.rows_map.ptr();
        ra.pair_pos = P.pair_pos.ptr(); ra.rows = m; ra.top = M.top; ra.experts = M.experts; ra.vocab = e->vocab;
        uzu_table_route_encode(cmd, &ra);
    }
    // a single expert takes every row in row order: its two products are plain ones (no row groups), so long passes run them on tcgen05
    const bool grouped = M.experts > 1;
    uzu_dense_linear_args up = gate_up_args();
    if (grouped) {
        up.batch = M.experts; up.w_z_stride = M.gate_up.stride();
        up.group_offsets = P.group_offsets.ptr(); up.rows_map = P.rows_map.ptr();
    }
    uzu_dense_linear_encode(cmd, &up);
    if (!paired) unit(m * M.top);
    // ... and, when its weight already sits on its input and no sublayer gate follows, its down projection adds straight into the residual
    const bool direct = !grouped && M.weight_on_input && !L.mlp_gate.present;
    uzu_dense_linear_args dn = dense_args(e, M.down, P.act.ptr(), m, direct ? P.resid.ptr() : P.pair_out.ptr());
    dn.lda = M.f; dn.accumulate = direct ? 1 : 0;
    if (grouped) {
        dn.batch = M.experts; dn.w_z_stride = M.down.stride();
        dn.group_offsets = P.group_offsets.ptr();
    }
    uzu_dense_linear_encode(cmd, &dn);
    if (direct) return;
    uzu_routed_combine_args ca{};
    ca.pairs = P.pair_out.ptr(); ca.pair_pos = P.pair_pos.ptr(); ca.output = P.resid.ptr(); ca.rows = m; ca.top = M.top; ca.n = W; ca.accumulate = 1;
    if (M.kind == GatedMlp::RoutedExperts) { ca.pair_weight = M.weight_on_input ? 0 : P.pair_weight.ptr(); ca.weight = 1.0f; }
    else ca.weight = 1.0f / (float)M.top;
    if (L.mlp_gate.present) {
        if (L.mlp_gate.bias.b) { ca.gate = P.proj2.ptr() + (uint64_t)L.mlp_gate.offset * 4; ca.gate_ld = M.router.rows; ca.gate_bias = L.mlp_gate.bias.ptr(); }
        if (L.mlp_gate.scale.b) ca.col_scale = L.mlp_gate.scale.ptr();
    }
    uzu_routed_combine_gated_encode(cmd, &ca);
}

static void encode_mixer(uzu_engine* e, uzu_command_buffer* cmd, const Layer& L, LayerState& S, const PassCtx& pc) {
    if (L.kind == MixGeneralDelta) encode_general_delta(e, cmd, L, S, pc);
    else if (L.kind == MixSigmoidAttention) encode_sigmoid_attention(e, cmd, L, S, pc);
    else if (L.kind == MixMinGru) encode_min_gru(e, cmd, L, S, pc);
    else if (L.kind == MixMlstm) encode_mlstm(e, cmd, L, S, pc);
    else if (L.has_window_attention() || L.has_retention()) encode_side_by_side(e, cmd, L, S, pc);
    else encode_latent_attention(e, cmd, L, S, pc);
}

static void set_norm(uzu_norm_add_args& a, const Norm& n, bool next) {
    if (next) { a.next_kind = n.kind; a.next_weight = n.scales.ptr(); a.next_bias = n.bias.ptr(); a.next_alpha = n.alpha; }
    else { a.kind = n.kind; a.weight = n.scales.ptr(); a.bias = n.bias.ptr(); a.alpha = n.alpha; }
}

// A sandwich layer: x <- x + mult * post(sublayer(pre(x))) for the mixer, the feed-forward (if any) and the token input (if any). A
// sublayer leaves its result in P.sub_out; ONE launch then norms it, adds it into the residual stream and norms the updated stream for
// whatever reads it next (the feed-forward, or the next layer's mixer: `next`; the pass's last layer leaves no normed copy).
// `normed_ready`: P.normed already holds this layer's normed input (the previous layer's last launch wrote it).
static void encode_sandwich_layer(uzu_engine* e, uzu_command_buffer* cmd, const Layer& L, LayerState& S, const PassCtx& pc, const Norm* next, bool normed_ready) {
    auto& P = e->pb;
    const uint32_t m = pc.m, W = e->model_dim;
    const bool has_mlp = L.gmlp.kind != GatedMlp::None;
    if (!normed_ready) {
        uzu_norm_add_args a{};
        a.input = P.resid.ptr(); a.output = P.normed.ptr(); a.rows = m; a.n = W; a.in_stride = W; a.epsilon = e->norm_eps;
        set_norm(a, L.pre_mixer, false);
        uzu_norm_add_encode(cmd, &a);
    }
    // residual += mult * norm(sub_out); then the norm of whoever reads the stream next, unless another addition comes first
    auto add = [&](const Norm& post, const Norm* reader) {
        uzu_norm_add_args a{};
        a.input = P.sub_out.ptr(); a.residual = P.resid.ptr(); a.rows = m; a.n = W; a.in_stride = W; a.epsilon = e->norm_eps; a.mult = L.residual_mult;
        set_norm(a, post, false);
        if (reader) { a.output = P.normed.ptr(); set_norm(a, *reader, true); }
        uzu_norm_add_encode(cmd, &a);
    };
    // Short passes (the decode step, short portions): a sublayer with ONE output projection and Dynamic Tanh norms around it takes the
    // norm, the add and the next norm as that projection's epilogue. Long passes keep the projection on the tensor-memory kernel and add
    // with a launch of their own.
    const bool fuse = m < 128 && L.kind != MixSideBySide;
    auto sublayer = [&](const Norm& post, const Norm* reader, auto&& encode) {
        const bool fused = fuse && post.kind == 1 && (!reader || reader->kind == 1);
        if (fused) { P.fused_post = &post; P.fused_reader = reader; P.fused_mult = L.residual_mult; }
        else P.redirect = true;
        encode();
        P.fused_post = P.fused_reader = nullptr;
        P.redirect = false;
        if (!fused) add(post, reader);
    };
    sublayer(L.post_mixer, has_mlp ? &L.pre_mlp : (L.side.present ? nullptr : next), [&] { encode_mixer(e, cmd, L, S, pc); });
    if (has_mlp) sublayer(L.post_mlp, L.side.present ? nullptr : next, [&] { encode_gated_mlp(e, cmd, L, pc, P.normed.ptr()); });
    if (L.side.present) {
        const TokenSide& T = L.side;
        if (m < 128) {   // the gate reads the residual stream itself; in short passes its epilogue forms gelu_tanh(.) * the token's table entries
            uzu_dense_linear_args x = dense_args(e, T.gate, P.resid.ptr(), m, P.lat.ptr());
            x.lda = W;
            x.token_ids = e->token_ids.ptr(); x.token_table = e->pb_side_embed.w.ptr(); x.token_gate_dt = e->store_dt;
            x.token_table_stride = e->pb_side_embed.cols; x.token_column = T.column; x.token_vocab = e->vocab;
            uzu_dense_linear_encode(cmd, &x);
        } else {         // long passes: the product on the tensor-memory kernel, then the unit
            encode_dense(e, cmd, T.gate, P.resid.ptr(), W, m, P.lat.ptr());
            uzu_token_gate_args ta{};
            ta.z = P.lat.ptr(); ta.token_ids = e->token_ids.ptr(); ta.table = e->pb_side_embed.w.ptr(); ta.out = P.lat.ptr();
            ta.rows = m; ta.n = T.dim; ta.vocab = e->vocab; ta.table_stride = e->pb_side_embed.cols; ta.column = T.column; ta.weights_dt = e->store_dt;
            uzu_token_gate_encode(cmd, &ta);
        }
        encode_dense(e, cmd, T.proj, P.lat.ptr(), T.dim, m, P.sub_out.ptr());
        Norm rms;
        rms.kind = 0; rms.scales = T.norm;
        add(rms, next);
    }
}

static void encode_parallel_block_decoder(uzu_engine* e, uzu_command_buffer* cmd, const PassCtx& pc, uint32_t row_begin, uint32_t row_end) {
    const uint32_t m = pc.m, W = e->model_dim;
    auto& P = e->pb;
    if (pc.trie) {
        cmd->record_error(UZU_ERROR_UNSUPPORTED, "speculation passes are not built for the parallel-block families");
        return;
    }
    uzu_embedding_f32_scaled_encode(cmd, e->token_ids.ptr(), e->pb_embed.w.ptr(), e->store_dt, P.resid.ptr(), m, e->vocab, W, e->input_scale);
    const bool dump = P.dump && !pc.dynamic && P.layer_dump.b;
    bool normed_ready = false;
    for (size_t i = 0; i < e->layers.size(); ++i) {
        Layer& L = e->layers[i];
        LayerState& S = e->state[i];
        if (L.sandwich) {
            const Norm* next = (i + 1 < e->layers.size() && e->layers[i + 1].sandwich) ? &e->layers[i + 1].pre_mixer : nullptr;
            encode_sandwich_layer(e, cmd, L, S, pc, next, normed_ready);
            normed_ready = next != nullptr;
            if (dump) uzu_command_buffer_encode_copy(cmd, P.resid.ptr(), P.layer_dump.ptr() + (uint64_t)i * MAX_ROWS * W * 4, (size_t)m * W * 4);
            continue;
        }
        uzu_group_rms_norm_args na{};
        na.input = P.resid.ptr(); na.scales = L.pre_mixer.scales.ptr(); na.output = P.normed.ptr();
        na.rows = m; na.n = W; na.groups = e->norm_groups; na.in_stride = W; na.out_stride = W; na.epsilon = e->norm_eps;
        const bool second = !L.sequential && L.pre_mlp.present && L.gmlp.kind != GatedMlp::None;      // the feed-forward norms the same x with its own weights
        if (second) { na.scales2 = L.pre_mlp.scales.ptr(); na.output2 = P.normed2.ptr(); }
        uzu_group_rms_norm_encode(cmd, &na);
        encode_mixer(e, cmd, L, S, pc);
        if (L.sequential && L.gmlp.kind != GatedMlp::None) {     // the feed-forward norms the residual the mixer has just added to
            uzu_group_rms_norm_args nb = na;
            nb.scales = L.pre_mlp.scales.ptr(); nb.scales2 = 0; nb.output2 = 0;
            uzu_group_rms_norm_encode(cmd, &nb);
        }
        if (L.gmlp.kind != GatedMlp::None) encode_gated_mlp(e, cmd, L, pc, second ? P.normed2.ptr() : P.normed.ptr());
        if (dump) uzu_command_buffer_encode_copy(cmd, P.resid.ptr(), P.layer_dump.ptr() + (uint64_t)i * MAX_ROWS * W * 4, (size_t)m * W * 4);
    }
    if (dump) P.dump_rows = m;
    encode_parallel_block_readout(e, cmd, row_begin, row_end);
}

static void encode_parallel_block_readout(uzu_engine* e, uzu_command_buffer* cmd, uint32_t row_begin, uint32_t row_end) {
    if (row_end <= row_begin) return;
    const uint32_t rows = row_end - row_begin, W = e->model_dim;
    auto& P = e->pb;
    if (e->pb_out_norm.present) {
        uzu_norm_add_args a{};
        a.input = P.resid.ptr() + (uint64_t)row_begin * W * 4; a.output = P.normed_rows.ptr(); a.rows = rows; a.n = W; a.in_stride = W; a.epsilon = e->norm_eps;
        set_norm(a, e->pb_out_norm, false);
        uzu_norm_add_encode(cmd, &a);
    } else {
        uzu_group_rms_norm_args na{};
        na.input = P.resid.ptr() + (uint64_t)row_begin * W * 4; na.scales = e->pb_final_norm.ptr(); na.output = P.normed_rows.ptr();
        na.rows = rows; na.n = W; na.groups = e->norm_groups; na.in_stride = W; na.out_stride = W; na.epsilon = e->norm_eps;
        uzu_group_rms_norm_encode(cmd, &na);
    }
    {
        uzu_dense_linear_args x = dense_args(e, e->pb_head, P.normed_rows.ptr(), rows, P.logits_f32.ptr());
        x.lda = W;
        if (e->has_logit_scale) x.scale = e->logit_scale;
        uzu_dense_linear_encode(cmd, &x);
    }
    uzu_logit_cap_f32_encode(cmd, P.logits_f32.ptr(), e->logits.ptr(), rows * e->vocab, e->logit_soft_cap, e->has_logit_soft_cap);
}
