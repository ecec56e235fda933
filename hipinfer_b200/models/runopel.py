"""The Runopel decoder as a ModelSpec: a token embedding into one or several residual streams; layers in the order
config.json lists them, each a pre-norm block (RMS norms) whose sublayers read a weighted sum of the streams and write
back into all of them while the streams are mixed (hyper-connections; with a residual multiplier); the mixer is the
state-space mixer with a scalar decay per head (a short causal convolution, a recurrent state per head, a gate before a
grouped norm) or latent attention (one cached latent and one rotated key part per token, a sliding window); the
feed-forward, where a layer has one, is dense with biases and limits or a mixture of experts with sigmoid scores that
multiply the experts' inputs; the model's norm over the sum of the streams, and a head tied to the embedding table with
a logit scale.

Tensor names: embed, final.norm, and per layer i under "l<i>.": norm1, norm2, hc1.in/out/mix, hc2.in/out/mix, mix.*,
mlp.* (experts under mlp.e<j>.*, the router mlp.router).
"""
from __future__ import annotations

from ..config.base import register_architecture
from ..config.runopel import RunopelConfig
from ..parts.spec import LayerSpec, ModelSpec, PartSpec, RunStep


def runopel_spec(c: RunopelConfig) -> ModelSpec:
    W, eps = c.width, c.norm_eps
    learned = c.streams is not None
    S = c.streams if learned else 1

    def norm(name, read=None):
        return PartSpec("streams_rmsnorm", dict(name=name, size=W, eps=eps, streams=S, read_name=read if learned else None))

    layers, order = [], []
    for i, L in enumerate(c.layers):
        m = L.mixer
        if L.type == "mamba2":
            mixer = PartSpec("mamba2", dict(hidden_size=W, heads=m.heads, vdim=m.vdim, state=m.state, groups=m.groups,
                                            norm_groups=m.norm_groups, conv=m.conv, eps=eps))
        else:
            mixer = PartSpec("latent_attention", dict(
                hidden_size=W, heads=m.heads, dim=m.dim, rot_dim=m.rot_dim, vdim=m.vdim, q_rank=None, kv_rank=m.kv_rank,
                scale=m.scale, eps=eps, rot_dims=m.rot.dims, rot_base=m.rot.base, gate=False, window=m.window))
        parts = dict(mixer_norm=norm("norm1", "hc1.in"), mixer=mixer)
        ff = L.mlp
        if ff is not None:
            parts["feed_forward_norm"] = norm("norm2", "hc2.in")
            if hasattr(ff, "experts"):
                parts["feed_forward"] = PartSpec("routed", dict(hidden_size=W, experts=ff.experts, top=ff.top, expert_size=ff.ff))
            else:
                parts["feed_forward"] = PartSpec("clamped_glu", dict(hidden_size=W, intermediate_size=ff.ff, limit=ff.limit))
        layers.append(LayerSpec(prefix=f"l{i}.", block="hyper_connections", parts=parts,
                                params=dict(hidden_size=W, streams=S, residual_mult=c.residual_mult, learned=learned)))
        order.append(RunStep(i))
    return ModelSpec(
        architecture=c.architecture, hidden_size=W, vocab_size=c.vocab, max_position=c.max_positions,
        embedding=PartSpec("token_streams", dict(name="embed", vocab_size=c.vocab, hidden_size=W, streams=S)),
        layers=tuple(layers), order=tuple(order), final_norm=norm("final.norm"),
        head=PartSpec("linear", dict(tied_to="embed", vocab_size=c.vocab, hidden_size=W, scale=c.logit_scale)),
        eos_token_ids=c.eos_token_ids)


register_architecture("Runopel", RunopelConfig, runopel_spec)
