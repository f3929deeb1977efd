"""A pure decode step as ONE kernel, when the model and the batch allow it.

The persistent decode kernel (``csrc/decode_persistent.cu``) runs embedding, every layer,
the final norm, the head and the greedy choice of a step in a single launch.  It serves one
shape of model: pre-norm blocks of LayerNorm, causal attention (heads of 64, no grouping, no
window, keys untouched by the position encoding) and a dense feed-forward, a token table with
a learned position table, a LayerNorm and a linear head at the end, one page group, bfloat16.
Whether a model has that shape is asked of its parts, not of its name: every standard part
answers ``fused_decode_params()`` with its tensors and constants (or ``None``), and
:func:`plan_fused_decode` puts the answers together — a model built from other parts simply
gets no plan and runs layer by layer.  A step takes the plan when it is made of single decoded
tokens only, at most sixteen.
"""

from __future__ import annotations

import torch

from .model import PreNormBlock


class FusedDecodePlan:
    """The descriptor records of one bound model on one runner's cache storage."""

    def __init__(self, model, ops, tables, sizes, parts):
        self.model, self.ops, self.tables = model, ops, tables
        self.sizes, self.parts = sizes, parts
        self.stop_after = 0        # tests: leave the kernel after so many phases (0: run it all)

    def applies(self, ctx) -> bool:
        plan = ctx.plan
        return (plan is not None and plan.single_new and plan.tile_cap == 0
                and 0 < plan.decode_cap and ctx.n_rows <= self.ops.FUSED_MAX_TOKENS
                and ctx.n_logit_rows <= self.ops.FUSED_MAX_TOKENS)

    def run(self, ctx):
        """Returns ``(logits, tokens)``: float32 ``[n_logit_rows, vocab]`` and the greedy tokens
        with the status word behind them (``[n_logit_rows + 1]`` int32)."""
        z, pr = self.sizes, self.parts
        T, W = ctx.n_rows, ctx.n_logit_rows
        x = ctx.buffer("residual", (T, z["width"]), torch.float32)
        qkv = ctx.buffer("qkv", (T, 3 * z["width"]), torch.bfloat16)
        att = ctx.buffer("attn_out", (T, z["width"]), torch.bfloat16)
        u = ctx.buffer("ff_inner", (T, z["inner"]), torch.bfloat16)
        logits = ctx.buffer("logits", (W, z["vocab"]), torch.float32) if W else None
        tokens = ctx.buffer(getattr(ctx, "tokens_name", "sampled"), (W + 1,), torch.int32)
        rn = ctx.runner
        pool = rn.storage.pools[0]
        self.ops.fused_decode(
            self.tables, wte=pr["wte"], wpe=pr["wpe"], lnf_g=pr["lnf_g"], lnf_b=pr["lnf_b"],
            eps_f=pr["eps_f"], width=z["width"], inner=z["inner"], vocab=z["vocab"],
            n_heads=z["n_heads"], pool=pool, num_pages=pool.shape[1],
            max_pages=ctx.tables[0].shape[1], x=x, qkv=qkv, att=att, u=u, logits=logits,
            tokens=tokens, feedback=ctx.feedback, tok_ids=ctx.tok_ids, tok_pos=ctx.tok_pos,
            tok_req=ctx.tok_req, table=ctx.tables[0], logit_rows=ctx.logit_rows,
            samp_slot=ctx.samp_slot, plan_head=ctx.plan.data, n_tokens=T,
            n_requests=ctx.n_requests, n_logit_rows=W, status=ctx.status,
            stop_after=self.stop_after)
        return logits, tokens


def plan_fused_decode(model, ops, storage, page_size: int):
    """A :class:`FusedDecodePlan` for a bound model, or None when some part of it (or the
    kernel interface in use) does not fit the persistent decode kernel."""
    if not hasattr(ops, "fused_decode_build") or model.dtype != torch.bfloat16:
        return None
    if len(model.cache_groups) != 1 or model.state_shapes or not model.capturable:
        return None
    emb = model.embedding.fused_decode_params()
    pos = model.position.fused_decode_params()
    fin = model.final_norm.fused_decode_params()
    head = model.head.fused_decode_params()
    if None in (emb, pos, fin, head):
        return None
    layers, sizes = [], None
    for call in model.schedule:
        block = model.blocks[call.layer]
        if type(block) is not PreNormBlock or not call.writes_cache:
            return None
        n1, mx = block.norm1.fused_decode_params(), block.mixer.fused_decode_params()
        n2, ff = block.norm2.fused_decode_params(), block.feed_forward.fused_decode_params()
        if None in (n1, mx, n2, ff):
            return None
        here = dict(width=mx["width"], inner=ff["inner"], n_heads=mx["n_heads"])
        if sizes is None:
            if not ops.fused_decode_supports(width=mx["width"], inner=ff["inner"],
                                             n_heads=mx["n_heads"], head_dim=mx["head_dim"],
                                             n_kv_heads=mx["n_kv_heads"], page_size=page_size,
                                             window=mx["window"]):
                return None
            sizes = here
        elif here != sizes or mx["head_dim"] * mx["n_heads"] != mx["width"] or mx["window"]:
            return None                 # the kernel takes layers of one size
        if ff["width"] != mx["width"] or n1["width"] != mx["width"] or n2["width"] != mx["width"]:
            return None
        gi, entry = model.entry_location[call.cache]
        layers.append(dict(
            w_qkv=mx["w_qkv"], b_qkv=mx["b_qkv"], w_out=mx["w_out"], b_out=mx["b_out"],
            w_fc=ff["w_in"], b_fc=ff["b_in"], w_mlp=ff["w_out"], b_mlp=ff["b_out"],
            ln1_g=n1["weight"], ln1_b=n1["bias"], eps1=n1["eps"],
            ln2_g=n2["weight"], ln2_b=n2["bias"], eps2=n2["eps"],
            scale=mx["scale"], act=ff["activation"], entry=entry))
    if sizes is None or emb["width"] != sizes["width"] or fin["width"] != sizes["width"]:
        return None
    if head["width"] != sizes["width"] or pos["width"] != sizes["width"]:
        return None
    sizes["vocab"] = head["vocab"]
    tables = ops.fused_decode_build(layers, head_weight=head["weight"], pool=storage.pools[0],
                                    width=sizes["width"], inner=sizes["inner"],
                                    vocab=sizes["vocab"])
    parts = dict(wte=emb["table"], wpe=pos["table"], lnf_g=fin["weight"], lnf_b=fin["bias"],
                 eps_f=fin["eps"])
    return FusedDecodePlan(model, ops, tables, sizes, parts)
