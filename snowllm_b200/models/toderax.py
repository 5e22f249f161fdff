"""Toderax as data: configuration -> ModelSpec.

A stack of pre-norm layers over several residual streams (block ``hyper``, norm ``group_rmsnorm``; without
``streams`` in the configuration: one stream and no learned stream weights).  The mixers are ``hgrn2`` (a gated
matrix memory) and ``side_by_side``: block-local softmax attention with sinks (``sink_attention``) beside a
retention memory (``retention``).  The feed-forward is softmax-routed experts with the clamped activation and a
shared expert (``routed_experts``), or none.  Tensor names: ``embed``, ``l<i>.norm{1,2}``, ``l<i>.hc{1,2}.{in,
out,mix}``, ``l<i>.mix.<what>`` (``l<i>.mix.{left,right}.<what>`` in a pair), ``l<i>.mlp.{router, e<j>.{gate,
up,down}, shared.{gate,up,down}}``, ``final.norm``, ``head``.  This file only names parts and passes them
their constants."""
from __future__ import annotations

from ..config.registry import register_architecture
from ..config.toderax import ARCHITECTURE, ToderaxConfig, read_toderax_config
from ..parts.spec import LayerSpec, ModelSpec, PartSpec, RunEntry


def toderax_model_spec(c: ToderaxConfig) -> ModelSpec:
    W, eps = c.width, c.norm_eps

    def norm(name):
        return PartSpec("group_rmsnorm", dict(size=W, eps=eps, groups=c.norm_groups), dict(weight=name))
    layers, run = [], []
    for i, layer in enumerate(c.layers):
        p, m = f"l{i}.mix.", layer.mixer
        if layer.type == "hgrn2":
            mixer = PartSpec("hgrn2", dict(hidden_size=W, num_heads=m["heads"], head_dim=m["dim"], v_head_dim=m["vdim"],
                                           head_norm_eps=eps),
                             dict(q_proj=p + "q", f_proj=p + "f", f_bias=p + "f.b", lower=p + "lower",
                                  v_proj=p + "v", norm=p + "norm", out_proj=p + "o"))
        else:
            l, r = m["left"], m["right"]
            lp, rp = p + "left.", p + "right."
            left = PartSpec("sink_attention",
                            dict(hidden_size=W, num_heads=l["heads"], num_kv_heads=l["kv_heads"], head_dim=l["dim"],
                                 v_head_dim=l["vdim"], scale=l["scale"], qk_norm_eps=eps, block=l["block"], biased=True),
                            dict(q_proj=lp + "q", k_proj=lp + "k", v_proj=lp + "v", out_proj=lp + "o",
                                 q_bias=lp + "q.b", k_bias=lp + "k.b", v_bias=lp + "v.b", temp=lp + "temp",
                                 sink=lp + "sink"))
            position = {"kind": "none"}
            if r["rot"] is not None:
                position = dict(kind="rope", head_dim=r["dim"], theta=r["rot"]["base"], rot_dim=r["rot"]["dims"])
            right = PartSpec("retention",
                             dict(hidden_size=W, num_heads=r["heads"], head_dim=r["dim"], v_head_dim=r["vdim"],
                                  head_norm_eps=eps, decay=tuple(r["decay"]), position=position),
                             dict(q_proj=rp + "q", k_proj=rp + "k", v_proj=rp + "v", gate_proj=rp + "g",
                                  out_proj=rp + "o"))
            mixer = PartSpec("side_by_side", dict(hidden_size=W, left=left, right=right, eps=eps, weights=(0.5, 0.5)),
                             dict(left_out=lp + "out", right_out=rp + "out"))
        ffn = ffn_norm = None
        if layer.mlp is not None:
            f, mlp = f"l{i}.mlp.", layer.mlp
            shared = None
            if mlp["shared"] is not None:
                shared = dict(intermediate_size=mlp["shared"]["ff"], limit=mlp["shared"]["limit"])
            ffn = PartSpec("routed_experts",
                           dict(hidden_size=W, intermediate_size=mlp["ff"], num_experts=mlp["experts"], top_k=mlp["top"],
                                norm_topk_prob=False, use_expert_bias=False, routed_scaling_factor=1.0,
                                scoring="softmax", activation="swish_clamp", limit=mlp["limit"], shared=shared),
                           dict(router=f + "router", experts=f + "e", expert_gate="gate", expert_up="up",
                                expert_down="down", fused_gate_up=f + "gate_up", fused_down=f + "down_all",
                                shared_gate=f + "shared.gate", shared_up=f + "shared.up",
                                shared_down=f + "shared.down"))
            ffn_norm = norm(f"l{i}.norm2")
        block = dict(streams=1, names=None)
        if c.streams is not None:
            hc = [{k: f"l{i}.hc{q}.{k}" for k in ("in", "out", "mix")} for q in ((1, 2) if ffn is not None else (1,))]
            block = dict(streams=c.streams, names=tuple(hc))
        layers.append(LayerSpec("hyper", mixer, ffn, norm(f"l{i}.norm1"), ffn_norm, block))
        run.append(RunEntry(i))
    embedding = PartSpec("embedding", dict(vocab_size=c.vocab, hidden_size=W, scale=c.embedding_scale),
                         dict(weight="embed"))
    head = PartSpec("linear_head", dict(vocab_size=c.vocab, hidden_size=W, tied=False), dict(weight="head"))
    return ModelSpec(architecture=c.architecture, vocab_size=c.vocab, hidden_size=W, embedding=embedding,
                     layers=layers, run=run, final_norm=norm("final.norm"), head=head)


register_architecture(ARCHITECTURE, read_toderax_config, toderax_model_spec)
