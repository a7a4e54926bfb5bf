"""Pifutar as a ModelSpec: a decoder whose layers mix with latent attention (a compressed cache, optionally
read from an earlier layer), retention or gated linear attention (a decaying matrix state), read every
sublayer's input through a short causal convolution, feed forward through a dense PolyNorm layer or a
mixture of experts chosen by a table of the token's id, and hand on a learned average of all layers' streams.
Norm weights are stored around zero; the head is the embedding table.

Tensor names: `embed`, `final.norm`, and per layer i `l<i>.norm1|norm2|canon1|canon2|dwa`, `l<i>.mix.*`,
`l<i>.mlp.*` (experts `l<i>.mlp.e<k>.gate|up|down`, shared expert `l<i>.mlp.shared.*`).
"""
from __future__ import annotations

from ..config.pifutar import PifutarConfig
from ..config.registry import register_architecture
from ..parts.spec import LayerSpec, ModelSpec, PartSpec, RunStep


def _rotary_name(base: float, dims: int) -> str:
    return f"rotary_{dims}_{base!r}"


def build_pifutar_spec(cfg: PifutarConfig) -> ModelSpec:
    D, V, eps = cfg.width, cfg.vocab, cfg.norm_eps
    n = len(cfg.layers)
    encodings = {}
    # the rows a latent-attention layer caches must outlive the widest window of the layers that read them
    cache_window = {}
    for i, l in enumerate(cfg.layers):
        if l.type == "latent_attention":
            src = i if l.mixer.kv_from is None else l.mixer.kv_from
            w = l.mixer.window
            cache_window[src] = w if src not in cache_window else (0 if 0 in (w, cache_window[src])
                                                                   else max(w, cache_window[src]))
    layers, order = [], []
    for i, l in enumerate(cfg.layers):
        p, m = f"l{i}.", l.mixer
        norm = lambda name: PartSpec("rmsnorm", dict(size=D, eps=eps, offset=1.0, output="float32"), dict(weight=name))
        conv = lambda name: PartSpec("causal_short_conv", dict(size=D, taps=cfg.taps), dict(weight=name))
        parts = {"mixer_norm": norm(p + "norm1"), "mixer_filter": conv(p + "canon1")}
        cache_from = None
        if l.type == "latent_attention":
            pe = None
            if m.rot_dims > 0:
                pe = _rotary_name(m.rot_base, m.rot_dims)
                encodings[pe] = PartSpec("rotary", dict(rot_dim=m.rot_dims, theta=m.rot_base, scaling=None,
                                                        layout="interleaved"))
            cache_from = m.kv_from
            parts["mixer"] = PartSpec("latent_attention", dict(
                hidden_size=D, num_heads=m.heads, head_dim=m.dim, rot_dim=m.rot_dim, value_dim=m.vdim,
                kv_rank=m.kv_rank, scale=m.scale, window=m.window,
                cache_window=cache_window[i if m.kv_from is None else m.kv_from], eps=eps,
                position_encoding=pe, shares_cache=m.kv_from is not None),
                dict(q=p + "mix.q", dkv=p + "mix.dkv", dkv_norm=p + "mix.dkv.norm", uk=p + "mix.uk",
                     uv=p + "mix.uv", o=p + "mix.o"))
        else:
            gated = l.type == "gla"
            parts["mixer"] = PartSpec("decay_linear_attention", dict(
                hidden_size=D, num_heads=m.heads, key_dim=m.dim, value_dim=m.vdim, eps=eps,
                decay=None if gated else list(m.decay), tau=m.tau, decay_rank=m.decay_rank,
                scale_on="q" if gated else "k", norm_weight=gated),
                dict(q=p + "mix.q", k=p + "mix.k", v=p + "mix.v", g=p + "mix.g", o=p + "mix.o", norm=p + "mix.norm",
                     a1=p + "mix.a1", a2=p + "mix.a2", a2_bias=p + "mix.a2.b"))
        f = l.mlp
        if f is not None:
            parts["ffn_norm"], parts["ffn_filter"] = norm(p + "norm2"), conv(p + "canon2")
            if f.kind == "dense":
                parts["ffn"] = PartSpec("polynorm_ff", dict(hidden_size=D, intermediate_size=f.ff, eps=eps),
                                        dict(up=p + "mlp.up", down=p + "mlp.down", act=p + "mlp.act"))
            else:
                parts["ffn"] = PartSpec("table_moe", dict(
                    hidden_size=D, vocab_size=V, num_experts=f.experts, top=f.top, intermediate_size=f.ff,
                    limit=f.limit, alpha=1.702, shift=1.0, shared_intermediate_size=f.shared_ff,
                    shared_limit=f.shared_limit),
                    dict(table=p + "mlp.table", gate=p + "mlp.e{e}.gate", up=p + "mlp.e{e}.up",
                         down=p + "mlp.e{e}.down", shared_gate=p + "mlp.shared.gate", shared_up=p + "mlp.shared.up",
                         shared_down=p + "mlp.shared.down", shared_sg=p + "mlp.shared.sg"))
        layers.append(LayerSpec("prenorm_depth_average", parts, dict(depth=i, levels=n + 1), dict(coef=p + "dwa")))
        order.append(RunStep(i, cache_from))
    embedding = PartSpec("token_embedding", dict(vocab_size=V, hidden_size=D), dict(weight="embed"))
    head = PartSpec("lm_head", dict(vocab_size=V, hidden_size=D, stored=False), dict(weight="embed"))
    return ModelSpec(
        hidden_size=D, vocab_size=V, max_position=cfg.max_position_embeddings, embedding=embedding, layers=layers,
        order=order, final_norm=PartSpec("rmsnorm", dict(size=D, eps=eps, offset=1.0), dict(weight="final.norm")),
        lm_head=head, position_encodings=encodings, eos_token_ids=cfg.eos_token_ids,
        # a layer without a feed-forward has no use for a second norm or convolution; a file may still hold them
        ignored_tensors=tuple(f"l{i}.{n}" for i, l in enumerate(cfg.layers) if l.mlp is None
                              for n in ("norm2", "canon2")))


register_architecture(PifutarConfig.ARCHITECTURE, PifutarConfig, build_pifutar_spec)
