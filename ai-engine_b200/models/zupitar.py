"""Zupitar as a ModelSpec: a decoder whose layers norm each sublayer's input and its output, mix with a state-space
mixer alone (`mamba2`) or side by side with an attention whose values are its keys (`parallel`: both read the same
input, their outputs are added with a weight each), and feed forward through a dense gated layer (relu) or a
mixture of experts chosen by a softmax router with a correction, groups and pass-through experts.  The head has a
tensor of its own and its logits are kept within +-logit_softcap by a tanh.

Tensor names: `embed`, `head`, `final.norm`, and per layer i `l<i>.norm1|norm1b|norm2|norm2b`; a state-space mixer
`<m>.in|conv|conv.b|dt_bias|A_log|D|norm|o` with <m> = `l<i>.mix` or `l<i>.mix.right`; the attention
`l<i>.mix.left.q|k|o|q.conv|k.conv`; `l<i>.mlp.gate|up|down`, or `l<i>.mlp.router|correction` and experts
`l<i>.mlp.e<k>.gate|up|down`.
"""
from __future__ import annotations

from ..config.registry import register_architecture
from ..config.zupitar import ZupitarConfig
from ..parts.spec import LayerSpec, ModelSpec, PartSpec, RunStep


def _rotary_name(a) -> str:
    return f"rotary_{a.rot_dims}_{a.rot_base!r}_{a.rot_factor!r}"


def build_zupitar_spec(cfg: ZupitarConfig) -> ModelSpec:
    D, V, eps = cfg.width, cfg.vocab, cfg.norm_eps
    encodings = {}
    layers = []

    def norm(name, post=False):
        # a post-norm reads a branch and hands its result to the float32 residual sum
        return PartSpec("rmsnorm", dict(size=D, eps=eps, output="float32" if post else None), dict(weight=name))

    def state_space(m, p):
        return PartSpec("scalar_decay_state_space", dict(
            hidden_size=D, num_heads=m.heads, value_dim=m.vdim, state_size=m.state, groups=m.groups, taps=m.conv,
            norm_groups=m.norm_groups, eps=eps),
            dict(conv=p + "conv", conv_bias=p + "conv.b", dt_bias=p + "dt_bias", a_log=p + "A_log", skip=p + "D",
                 norm=p + "norm", o=p + "o", **{"in": p + "in"}))

    for i, l in enumerate(cfg.layers):
        p = f"l{i}."
        parts = {"mixer_norm": norm(p + "norm1"), "mixer_post_norm": norm(p + "norm1b", post=True)}
        if l.type == "parallel":
            a = l.left
            pe = None
            if a.rot_dims > 0:
                pe = _rotary_name(a)
                encodings[pe] = PartSpec("rotary", dict(
                    rot_dim=a.rot_dims, theta=a.rot_base,
                    scaling=dict(type="linear", factor=a.rot_factor) if a.rot_factor != 1.0 else None))
            q = p + "mix.left."
            left = PartSpec("gqa_attention", dict(
                hidden_size=D, num_heads=a.heads, num_kv_heads=a.kv_heads, head_dim=a.dim, window=0, scale=a.scale,
                position_encoding=pe, qk_conv=a.conv, tied_values=True),
                dict(q=q + "q", k=q + "k", o=q + "o", q_conv=q + "q.conv", k_conv=q + "k.conv"))
            parts["mixer"] = PartSpec("parallel_mixers", dict(
                left=left, right=state_space(l.right, p + "mix.right."), left_scale=l.left_scale,
                right_scale=l.right_scale))
        else:
            parts["mixer"] = state_space(l.right, p + "mix.")
        f = l.mlp
        if f is not None:
            parts["ffn_norm"], parts["ffn_post_norm"] = norm(p + "norm2"), norm(p + "norm2b", post=True)
            if f.kind == "dense":
                parts["ffn"] = PartSpec("swiglu", dict(hidden_size=D, intermediate_size=f.ff, activation="relu"),
                                        dict(gate=p + "mlp.gate", up=p + "mlp.up", down=p + "mlp.down"))
            else:
                parts["ffn"] = PartSpec("routed_moe", dict(
                    hidden_size=D, num_experts=f.experts, identity=f.identity, top=f.top, intermediate_size=f.ff,
                    groups=f.group_count, keep=f.group_keep, activation="silu"),
                    dict(router=p + "mlp.router", correction=p + "mlp.correction", gate=p + "mlp.e{e}.gate",
                         up=p + "mlp.e{e}.up", down=p + "mlp.e{e}.down"))
        layers.append(LayerSpec("sandwich_norm", parts))
    embedding = PartSpec("token_embedding", dict(vocab_size=V, hidden_size=D), dict(weight="embed"))
    head = PartSpec("lm_head", dict(vocab_size=V, hidden_size=D, softcap=cfg.logit_softcap), dict(weight="head"))
    return ModelSpec(
        hidden_size=D, vocab_size=V, max_position=cfg.max_position_embeddings, embedding=embedding, layers=layers,
        order=[RunStep(i) for i in range(len(layers))], final_norm=PartSpec("rmsnorm", dict(size=D, eps=eps),
                                                                            dict(weight="final.norm")),
        lm_head=head, position_encodings=encodings, eos_token_ids=cfg.eos_token_ids,
        # a layer without a feed-forward has no use for its two norms; a file may still hold them
        ignored_tensors=tuple(f"l{i}.{n}" for i, l in enumerate(cfg.layers) if l.mlp is None
                              for n in ("norm2", "norm2b")))


register_architecture(ZupitarConfig.ARCHITECTURE, ZupitarConfig, build_zupitar_spec)
