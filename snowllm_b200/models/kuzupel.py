"""Kuzupel as data: configuration -> ModelSpec.

A stack of pre-norm layers whose sublayers enter the residual stream times a constant (block ``prenorm`` with
``residual_scale``, norm ``rmsnorm``).  The embedding adds a row of a second table chosen by a hash of the
token and the one before it (``pair_hash_embedding``).  The mixers are ``slope_attention`` (a window, q and k
normalised over the whole projection, a distance penalty per head) and ``conv_gate_attention`` (convolved
projections, per-head norms, partial rotation, a window beside the first positions, one more term in the
softmax's sum, gated heads).  The feed-forward is the clamped gated form, dense (``gated``) or as routed
experts whose weights are the softmax over the picked logits, with a shared expert behind a gate per token
(``routed_experts``), or none.  The head caps its logits.  Tensor names: ``embed``, ``bigram``,
``l<i>.norm{1,2}``, ``l<i>.mix.{q,k,v,o,g}``, ``l<i>.mix.{q,k}.norm``, ``l<i>.mix.{q,k,v}.conv``,
``l<i>.mlp.{gate,up,down}`` or ``l<i>.mlp.{router, router.b, e<j>.{gate,up,down}, shared.{gate,up,down,sg}}``,
``final.norm``, ``head``.  This file only names parts and passes them their constants."""
from __future__ import annotations

from ..config.kuzupel import ARCHITECTURE, KuzupelConfig, read_kuzupel_config
from ..config.registry import register_architecture
from ..parts.spec import LayerSpec, ModelSpec, PartSpec, RunEntry

SLOPE_RANGE = 8.0        # the heads' distance slopes are 2^(-SLOPE_RANGE * (h + 1) / heads)


def kuzupel_model_spec(c: KuzupelConfig) -> ModelSpec:
    W, eps = c.width, c.norm_eps

    def norm(name):
        return PartSpec("rmsnorm", dict(size=W, eps=eps), dict(weight=name))
    layers, run = [], []
    for i, layer in enumerate(c.layers):
        p, m = f"l{i}.mix.", layer.mixer
        common = dict(hidden_size=W, num_heads=m["heads"], num_kv_heads=m["kv_heads"], head_dim=m["dim"],
                      v_head_dim=m["vdim"], scale=m["scale"], qk_norm_eps=eps, window=m["window"])
        names = dict(q_proj=p + "q", k_proj=p + "k", v_proj=p + "v", out_proj=p + "o", q_norm=p + "q.norm",
                     k_norm=p + "k.norm")
        if layer.type == "attention":
            mixer = PartSpec("slope_attention", dict(common, slope_range=SLOPE_RANGE, keep_first=m["keep_first"]),
                             names)
        else:
            position = {"kind": "none"}
            if m["rot"] is not None:
                position = dict(kind="rope", head_dim=m["dim"], theta=m["rot"]["base"], rot_dim=m["rot"]["dims"],
                                precise=True)
            mixer = PartSpec("conv_gate_attention",
                             dict(common, conv_taps=m["conv"], keep_first=m["keep_first"], one_more=True,
                                  position=position),
                             dict(names, gate_proj=p + "g", q_conv=p + "q.conv", k_conv=p + "k.conv",
                                  v_conv=p + "v.conv"))
        ffn = ffn_norm = None
        if layer.mlp is not None:
            f, mlp = f"l{i}.mlp.", layer.mlp
            if mlp["kind"] == "dense":
                ffn = PartSpec("gated", dict(hidden_size=W, intermediate_size=mlp["ff"], activation="swish_clamp",
                                             limit=mlp["limit"]),
                               dict(gate=f + "gate", up=f + "up", down=f + "down"))
            else:
                shared = None
                if mlp["shared"] is not None:
                    shared = dict(intermediate_size=mlp["shared"]["ff"], limit=mlp["shared"]["limit"], row_gate=True)
                ffn = PartSpec("routed_experts",
                               dict(hidden_size=W, intermediate_size=mlp["ff"], num_experts=mlp["experts"],
                                    top_k=mlp["top"], norm_topk_prob=False, use_expert_bias=True,
                                    routed_scaling_factor=1.0, scoring="softmax_picked", activation="swish_clamp",
                                    limit=mlp["limit"], shared=shared),
                               dict(router=f + "router", expert_bias=f + "router.b", experts=f + "e",
                                    expert_gate="gate", expert_up="up", expert_down="down",
                                    fused_gate_up=f + "gate_up", fused_down=f + "down_all",
                                    shared_gate=f + "shared.gate", shared_up=f + "shared.up",
                                    shared_down=f + "shared.down", shared_row_gate=f + "shared.sg"))
            ffn_norm = norm(f"l{i}.norm2")
        layers.append(LayerSpec("prenorm", mixer, ffn, norm(f"l{i}.norm1"), ffn_norm,
                                dict(residual_scale=c.residual_mult)))
        run.append(RunEntry(i))
    if c.pair_table is not None:
        embedding = PartSpec("pair_hash_embedding",
                             dict(vocab_size=c.vocab, hidden_size=W, scale=c.embedding_scale, **c.pair_table),
                             dict(weight="embed", pairs="bigram"))
    else:
        embedding = PartSpec("embedding", dict(vocab_size=c.vocab, hidden_size=W, scale=c.embedding_scale),
                             dict(weight="embed"))
    head = PartSpec("linear_head", dict(vocab_size=c.vocab, hidden_size=W, tied=False, softcap=c.logit_softcap),
                    dict(weight="head"))
    return ModelSpec(architecture=c.architecture, vocab_size=c.vocab, hidden_size=W, embedding=embedding,
                     layers=layers, run=run, final_norm=norm("final.norm"), head=head)


register_architecture(ARCHITECTURE, read_kuzupel_config, kuzupel_model_spec)
