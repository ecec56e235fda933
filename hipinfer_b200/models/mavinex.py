"""The Mavinex decoder as a ModelSpec: a scaled token embedding; layers in the order config.json lists them, each with the
norm AFTER the sum, x <- norm1(alpha * x + mixer(x)) and, where the layer has a feed-forward, x <- norm2(alpha * x + ff(x)),
RMS norms whose weight is stored around zero (the row is multiplied by 1 + w). The mixer is either two mixers side by side
whose results are normed and averaged (grouped-query attention with a sliding window, an RMS norm over the whole query
and key rows before the interleaved rotation with frequencies rescaled by wavelength bands, an output gate per element;
beside it the selective state-space mixer), or latent attention (one cached latent and one rotated key part per token, a
sliding window, the rotate-half pairing with YaRN scaling, a sink in the softmax, an output gate per head). The
feed-forward is a mixture of experts whose largest router logits (with a bias) choose and whose weights are the softmax
over the chosen logits. A layer may run with the tensors of another layer and a cache and state of its own. The model's
norm and an untied head.

Tensor names: embed, final.norm, head, and per layer i under "l<i>.": norm1, norm2, mix.* (a parallel layer: mix.left.*,
mix.right.*, mix.left.out, mix.right.out), mlp.router, mlp.router.b, mlp.e<j>.gate / .up / .down.
"""
from __future__ import annotations

from ..config.base import register_architecture
from ..config.mavinex import MavinexConfig
from ..parts.spec import LayerSpec, ModelSpec, PartSpec, RunStep


def _scaling(rot, kind):
    sc = rot.scaling_dict()
    return dict(sc, kind=kind) if sc else None


def _layer_spec(c: MavinexConfig, L, prefix: str) -> LayerSpec:
    W, eps = c.width, c.norm_eps
    m = L.mixer
    if L.type == "parallel":
        a, b = m.left, m.right
        left = PartSpec("masked_attention", dict(
            hidden_size=W, heads=a.heads, kv_heads=a.kv_heads, dim=a.dim, vdim=a.vdim, scale=a.scale, eps=eps,
            rot_dims=a.rot.dims, rot_base=a.rot.base, rot_scaling=_scaling(a.rot, "wavelength_bands"), pairing="interleaved",
            row_norm=True, mask="window" if a.window else "causal", window=a.window or 0, gate="element",
            q_name="mix.left.q", k_name="mix.left.k", v_name="mix.left.v", g_name="mix.left.g", o_name="mix.left.o",
            q_norm_name="mix.left.q.norm", k_norm_name="mix.left.k.norm"))
        right = PartSpec("selective_scan", dict(
            hidden_size=W, inner=b.inner, state=b.state, dt_rank=b.dt_rank, conv=b.conv,
            in_name="mix.right.in", conv_name="mix.right.conv", conv_bias_name="mix.right.conv.b", x_name="mix.right.x",
            dt_name="mix.right.dt", dt_bias_name="mix.right.dt.b", a_log_name="mix.right.A_log", d_name="mix.right.D",
            o_name="mix.right.o"))
        mixer = PartSpec("side_by_side", dict(hidden_size=W, left=left, right=right, eps=eps, mix=0.5,
                                              left_norm_name="mix.left.out", right_norm_name="mix.right.out"))
    else:
        mixer = PartSpec("latent_attention", dict(
            hidden_size=W, heads=m.heads, dim=m.dim, rot_dim=m.rot_dim, vdim=m.vdim, q_rank=None, kv_rank=m.kv_rank,
            scale=m.scale, eps=eps, rot_dims=m.rot.dims, rot_base=m.rot.base, rot_scaling=_scaling(m.rot, "yarn"),
            pairing="half", gate="head", window=m.window, sink=True))
    norm = lambda name: PartSpec("rmsnorm", dict(name=name, size=W, eps=eps, one_plus=True))
    parts = dict(mixer=mixer, mixer_norm=norm("norm1"))
    if L.mlp is not None:
        parts["feed_forward"] = PartSpec("routed", dict(hidden_size=W, experts=L.mlp.experts, top=L.mlp.top, expert_size=L.mlp.ff,
                                                        score="softmax_chosen", weight_at="output", router_bias=True))
        parts["feed_forward_norm"] = norm("norm2")
    return LayerSpec(prefix=prefix, block="post_norm", parts=parts, params=dict(hidden_size=W, alpha=c.postln_alpha))


def mavinex_spec(c: MavinexConfig) -> ModelSpec:
    layers, order, index = [], [], {}
    for i, L in enumerate(c.layers):
        j = c.weights_layer(i)
        # a layer that runs with another layer's tensors is that layer's parts run again (a cache and state of its own),
        # unless its entry differs from the other's: then it gets parts of its own over the same tensors
        key = (j, L.type, L.mixer, L.mlp)
        if key not in index:
            index[key] = len(layers)
            layers.append(_layer_spec(c, L, f"l{j}."))
        order.append(RunStep(index[key]))
    W = c.width
    return ModelSpec(
        architecture=c.architecture, hidden_size=W, vocab_size=c.vocab, max_position=c.max_positions,
        embedding=PartSpec("token_position", dict(name="embed", vocab_size=c.vocab, hidden_size=W, scale=c.embedding_scale)),
        layers=tuple(layers), order=tuple(order),
        final_norm=PartSpec("rmsnorm", dict(name="final.norm", size=W, eps=c.norm_eps, one_plus=True)),
        head=PartSpec("linear", dict(name="head", vocab_size=c.vocab, hidden_size=W)),
        eos_token_ids=c.eos_token_ids)


register_architecture("Mavinex", MavinexConfig, mavinex_spec)
