"""BERT pre-training (masked-LM + next-sentence) as one leaf module.

Architecture of the reference's benchmark model
(``examples/benchmark/utils/modeling/networks/transformer_encoder.py:111-169``,
``layers/transformer.py:206-246`` post-LN blocks with tanh-GELU,
``networks/masked_lm.py:64-92``, ``networks/classification.py:61-68``, loss
``bert_models.py:115-138``). ``BertConfig`` defaults are BERT-large.

Two execution paths over the same parameters:

* ``reference_loss`` - plain PyTorch ops in fp32; runs anywhere; the numerics
  oracle for the kernels and the path CPU ranks use.
* the fused path (CUDA, after ``materialize``) - forward **and** backward are
  explicit sequences of the hand-written sm_100a kernels: tcgen05 GEMMs (the
  backward products read the forward tensors as MN-major operands, so nothing is
  transposed), attention as batched tcgen05 GEMMs over strided views of the
  fused QKV projection, fused bias/GELU/residual epilogues, layernorm /
  softmax / cross-entropy kernels. Gradients are written straight into the flat
  fp32 gradient buffer; ``grad_ready`` is called as parameter ranges complete so
  that the engine can start their all-reduce while the rest of the backward
  pass still runs.

The MLM output projection is untied from the word embeddings by default
(``tie_word_embeddings=False``): then the word-embedding gradient is purely
row-sparse and a Parallax strategy can route it through the sparse
parameter-server path, which the reference's tied head makes dense
(``networks/masked_lm.py:56,76-78``).
"""
import math
import os
import json
from dataclasses import asdict, dataclass, fields

import torch
from torch import nn
import torch.nn.functional as F

from autodist_b200.ops.flat import FlatParams

EPI_NONE, EPI_BIAS, EPI_BIAS_GELU, EPI_MUL_GELU_GRAD, EPI_ADD, EPI_BIAS_TANH = range(6)


@dataclass
class BertConfig:
    vocab_size: int = 30522
    hidden_size: int = 1024
    num_hidden_layers: int = 24
    num_attention_heads: int = 16
    intermediate_size: int = 4096
    max_position_embeddings: int = 512
    type_vocab_size: int = 2
    hidden_dropout_prob: float = 0.1
    attention_probs_dropout_prob: float = 0.1
    initializer_range: float = 0.02
    layer_norm_eps: float = 1e-12
    tie_word_embeddings: bool = False

    @classmethod
    def large(cls, **kw):
        return cls(**kw)

    # JSON round trip in the layout of the published ``bert_config.json`` files
    # (reference: ``examples/benchmark/utils/bert_modeling.py:86-108``); unknown keys are ignored.
    @classmethod
    def from_dict(cls, obj):
        known = {f.name for f in fields(cls)}
        return cls(**{k: v for k, v in obj.items() if k in known})

    @classmethod
    def from_json_file(cls, path):
        with open(path) as f:
            return cls.from_dict(json.load(f))

    def to_dict(self):
        return asdict(self)

    def to_json_string(self):
        return json.dumps(self.to_dict(), indent=2, sort_keys=True) + "\n"

    @classmethod
    def base(cls, **kw):
        return cls(hidden_size=768, num_hidden_layers=12, num_attention_heads=12, intermediate_size=3072, **kw)

    @classmethod
    def tiny(cls, **kw):
        d = dict(vocab_size=1000, hidden_size=128, num_hidden_layers=2, num_attention_heads=2, intermediate_size=256,
                 max_position_embeddings=128)
        d.update(kw)
        return cls(**d)


class BertPretrainer(nn.Module):
    _autodist_leaf = True

    def __init__(self, config: BertConfig):
        super().__init__()
        c = self.config = config
        H, Fd = c.hidden_size, c.intermediate_size
        std = c.initializer_range

        def w(*shape):
            return nn.Parameter(torch.randn(*shape) * std)

        def zeros(*shape):
            return nn.Parameter(torch.zeros(*shape))

        def ones(*shape):
            return nn.Parameter(torch.ones(*shape))

        P = nn.ParameterDict
        self.emb = P({"word": w(c.vocab_size, H), "pos": w(c.max_position_embeddings, H), "tok_type": w(c.type_vocab_size, H),
                      "ln_g": ones(H), "ln_b": zeros(H)})
        self.layers = nn.ModuleList([
            P({"qkv_w": w(3 * H, H), "qkv_b": zeros(3 * H), "out_w": w(H, H), "out_b": zeros(H),
               "ln1_g": ones(H), "ln1_b": zeros(H), "w1": w(Fd, H), "b1": zeros(Fd), "w2": w(H, Fd), "b2": zeros(H),
               "ln2_g": ones(H), "ln2_b": zeros(H)}) for _ in range(c.num_hidden_layers)])
        self.pooler = P({"w": w(H, H), "b": zeros(H)})
        self.nsp = P({"w": w(2, H), "b": zeros(2)})
        mlm = {"dense_w": w(H, H), "dense_b": zeros(H), "ln_g": ones(H), "ln_b": zeros(H), "bias": zeros(c.vocab_size)}
        if not c.tie_word_embeddings:
            mlm["decoder_w"] = w(c.vocab_size, H)
        self.mlm = P(mlm)
        self.flat = None
        self.grad_ready = None          # callable(lo, hi) set by the engine
        self._ws = None
        self._seed = 0x5EED
        self.training_dropout = True
        # S == 128: softmax inside the QK^T / dP GEMM epilogues. Measured slower than the stand-alone softmax kernels
        # (20.9 vs 20.1 ms per BERT-large step: a 64-deep contraction cannot hide a 128-exponential epilogue), so off.
        self.fused_attention_softmax = False
        # Bias gradients (column sums) on a side stream next to the weight-gradient GEMMs instead of between them.
        self.side_stream_bias_grads = os.environ.get("AUTODIST_BERT_SIDE_STREAM", "1") == "1"

    def sparse_grad_parameters(self):
        """Variables whose gradient is row-sparse (only when the output projection is untied)."""
        return [] if self.config.tie_word_embeddings else [self.emb["word"]]

    def sparse_lookup_parameters(self):
        """Tables the fused path reads row by row, so that an engine may keep them as one row shard per rank."""
        return self.sparse_grad_parameters()

    # ------------------------------------------------------------------ reference path (plain PyTorch, fp32)
    def reference_loss(self, input_ids, input_mask, segment_ids, mlm_positions, mlm_ids, mlm_weights, nsp_labels,
                       dropout=False):
        c = self.config
        B, S = input_ids.shape
        H, nh = c.hidden_size, c.num_attention_heads
        D = H // nh
        e = self.emb
        x = e["word"][input_ids] + e["pos"][:S][None] + e["tok_type"][segment_ids]
        x = F.layer_norm(x, (H,), e["ln_g"], e["ln_b"], c.layer_norm_eps)
        add_mask = (1.0 - input_mask.to(x.dtype))[:, None, None, :] * -10000.0
        pd_h = c.hidden_dropout_prob if dropout else 0.0
        pd_a = c.attention_probs_dropout_prob if dropout else 0.0
        for L in self.layers:
            qkv = F.linear(x, L["qkv_w"], L["qkv_b"]).view(B, S, 3, nh, D)
            q, k, v = (qkv[:, :, i].permute(0, 2, 1, 3) for i in range(3))
            p = torch.softmax(q @ k.transpose(-1, -2) / math.sqrt(D) + add_mask, -1)
            p = F.dropout(p, pd_a, dropout)
            ctx = (p @ v).permute(0, 2, 1, 3).reshape(B, S, H)
            ao = F.dropout(F.linear(ctx, L["out_w"], L["out_b"]), pd_h, dropout)
            x = F.layer_norm(ao + x, (H,), L["ln1_g"], L["ln1_b"], c.layer_norm_eps)
            g = F.gelu(F.linear(x, L["w1"], L["b1"]), approximate="tanh")
            fo = F.dropout(F.linear(g, L["w2"], L["b2"]), pd_h, dropout)
            x = F.layer_norm(fo + x, (H,), L["ln2_g"], L["ln2_b"], c.layer_norm_eps)
        pooled = torch.tanh(F.linear(x[:, 0], self.pooler["w"], self.pooler["b"]))
        nsp_logits = F.linear(pooled, self.nsp["w"], self.nsp["b"])
        nsp_loss = F.cross_entropy(nsp_logits, nsp_labels.view(-1))
        m = self.mlm
        flat_pos = (mlm_positions + torch.arange(B, device=x.device)[:, None] * S).view(-1)
        xm = x.reshape(B * S, H)[flat_pos]
        hm = F.gelu(F.linear(xm, m["dense_w"], m["dense_b"]), approximate="tanh")
        hm = F.layer_norm(hm, (H,), m["ln_g"], m["ln_b"], c.layer_norm_eps)
        dec = e["word"] if c.tie_word_embeddings else m["decoder_w"]
        logits = F.linear(hm, dec, m["bias"])
        per = F.cross_entropy(logits, mlm_ids.view(-1), reduction="none")
        wts = mlm_weights.view(-1).to(per.dtype)
        mlm_loss = (per * wts).sum() / (wts.sum() + 1e-5)
        return mlm_loss + nsp_loss

    # ------------------------------------------------------------------ fused path
    def materialize(self, device, grad_alloc=None, master_alloc=None, p16_alloc=None):
        """Move the parameters into flat master / bf16 / gradient buffers on ``device``."""
        named = [(n, p) for n, p in self.named_parameters()]
        self.flat = FlatParams(named, device, grad_alloc, master_alloc=master_alloc, p16_alloc=p16_alloc)
        self._ws = None
        return self.flat

    def _workspace(self, B, S, P):
        key = (B, S, P)
        if self._ws is not None and self._ws["key"] == key:
            return self._ws
        from autodist_b200 import ops
        E = ops.ext(required=True)
        c = self.config
        dev = self.flat.device
        T, H, Fd, nh = B * S, c.hidden_size, c.intermediate_size, c.num_attention_heads
        V = c.vocab_size
        Vp = (V + 7) // 8 * 8

        def bf(*shape):
            return torch.empty(*shape, dtype=torch.bfloat16, device=dev)

        def f32(*shape):
            return torch.empty(*shape, dtype=torch.float32, device=dev)

        drop_a = c.attention_probs_dropout_prob > 0 and self.training_dropout
        layers = []
        for _ in range(c.num_hidden_layers):
            layers.append({
                "qkv": bf(T, 3 * H), "p": bf(B, nh, S, S), "pd": bf(B, nh, S, S) if drop_a else None,
                "ctx": bf(T, H), "z1": bf(T, H), "m1": f32(T), "r1": f32(T), "x1": bf(T, H),
                "u": bf(T, Fd), "g": bf(T, Fd), "z2": bf(T, H), "m2": f32(T), "r2": f32(T), "out": bf(T, H)})
        n_part = max( E.colsum_parts(T) * max(4 * H, Fd, 3 * H, 2 * H),
                     E.colsum_parts(B * P) * Vp)
        ws = {
            "key": key, "E": E, "layers": layers, "Vp": Vp,
            "z0": bf(T, H), "m0": f32(T), "r0": f32(T), "x0": bf(T, H), "mask": f32(B, S),
            "tmp": bf(T, H), "scores": bf(B, nh, S, S),
            # backward scratch
            "d_a": bf(T, H), "d_b": bf(T, H), "d_c": bf(T, H), "d_big": bf(T, Fd), "d_qkv": bf(T, 3 * H),
            "d_p": bf(B, nh, S, S), "part": f32(n_part),
            "ln_part": torch.zeros(E.ln_bwd_part_floats(H), dtype=torch.float32, device=dev),     # zero between calls by contract
            # bias gradients are column sums that nothing in the layer waits for: they run on a side stream next to the
            # GEMMs, each with its own partial-sum scratch (joined before the layer's gradients are reported ready)
            "side_part": [f32(E.colsum_parts(T) * max(Fd, 3 * H)) for _ in range(4)],
            "side_stream": torch.cuda.Stream(device=dev), "side_fork": torch.cuda.Event(), "side_join": torch.cuda.Event(),
            # heads
            "pooled": bf(B, H), "nsp_logits": bf(B, 8), "d_pooled": bf(B, H), "d_pre": bf(B, H),
            "flat_pos": torch.empty(B * P, dtype=torch.int64, device=dev),
            "row_index": torch.arange(T, dtype=torch.int64, device=dev),
            "xm": bf(B * P, H), "hm_u": bf(B * P, H), "hm": bf(B * P, H), "hl": bf(B * P, H), "mm": f32(B * P),
            "mr": f32(B * P), "logits": bf(B * P, Vp), "d_hl": bf(B * P, H), "d_hm": bf(B * P, H), "d_hu": bf(B * P, H),
            "d_xm": bf(B * P, H), "d_bias": f32(Vp),
            "loss": torch.zeros(1, dtype=torch.float32, device=dev), "denom": f32(1), "one": torch.ones(1, device=dev),
            "err": torch.zeros(1, dtype=torch.int32, device=dev),
            "step": torch.zeros(1, dtype=torch.int64, device=dev),
        }
        self._ws = ws
        return ws

    def _gemm(self, ws, a, b, c, a_mn=False, b_mn=False, epi=EPI_NONE, bias=None, c2=None, aux=None, alpha=1.0, beta=0.0, bn=0):
        ws["E"].gemm(a, b, c, a_mn, b_mn, epi, bias, c2, aux, alpha, beta, ws["err"], bn)

    def fused_forward_backward(self, input_ids, input_mask, segment_ids, mlm_positions, mlm_ids, mlm_weights, nsp_labels,
                               backward=True):
        """Loss (device scalar) of one batch; with ``backward`` the flat gradient buffer is filled as well."""
        c, fl = self.config, self.flat
        B, S = input_ids.shape
        if B == 0:
            raise ValueError("this replica received an empty batch: feed at least one sequence per replica of the node")
        P = mlm_positions.shape[1]
        ws = self._workspace(B, S, P)
        E = ws["E"]
        T, H, Fd, nh = B * S, c.hidden_size, c.intermediate_size, c.num_attention_heads
        D = H // nh
        V, Vp = c.vocab_size, ws["Vp"]
        w16, w32, g = fl.w16, fl.w32, fl.g
        eps = c.layer_norm_eps
        drop = self.training_dropout and backward
        ph = c.hidden_dropout_prob if drop else 0.0
        pa = c.attention_probs_dropout_prob if drop else 0.0
        step = ws["step"]
        gm = lambda *a, **k: self._gemm(ws, *a, **k)   # noqa: E731
        seed = lambda l, site: self._seed + 64 * l + site   # noqa: E731
        scale = 1.0 / math.sqrt(D)
        fused_sm = S == 128 and self.fused_attention_softmax

        ids = input_ids.reshape(-1)
        tts = segment_ids.reshape(-1)
        ws["loss"].zero_()
        E.increment(step)
        ws["mask"].copy_((1.0 - input_mask.to(torch.float32)) * -10000.0)

        def heads_view(t, i):          # [T, 3H] -> [B, nh, S, D] view of q (0), k (1) or v (2)
            return t.view(B, S, 3, nh, D)[:, :, i].permute(0, 2, 1, 3)

        def ctx_view(t):               # [T, H] -> [B, nh, S, D]
            return t.view(B, S, nh, D).permute(0, 2, 1, 3)

        # ------------------------------ forward
        word_rows = getattr(self.emb["word"], "_sparse_rows", None)
        if word_rows is not None:
            # sharded table: the rows of this batch are fetched from the shards that own them (peer memory)
            rows = word_rows.lookup(ids)
            E.embed_sum(rows, w16["emb.pos"], w16["emb.tok_type"], ws["row_index"], tts, ws["z0"], S, ws["err"])
        else:
            E.embed_sum(w16["emb.word"], w16["emb.pos"], w16["emb.tok_type"], ids, tts, ws["z0"], S, ws["err"])
        E.ln_fwd(ws["z0"], None, w32["emb.ln_g"], w32["emb.ln_b"], None, ws["x0"], ws["m0"], ws["r0"], eps, 0.0, 0, None)
        x = ws["x0"]
        for l, A in enumerate(ws["layers"]):
            n = f"layers.{l}."
            gm(x, w16[n + "qkv_w"], A["qkv"], epi=EPI_BIAS, bias=w32[n + "qkv_b"])
            q, k, v = (heads_view(A["qkv"], i) for i in range(3))
            if fused_sm:      # scores never leave the SM: scale, mask, softmax and dropout run in the GEMM epilogue
                E.gemm_softmax(q, k, A["p"], A["pd"] if pa > 0 else None, ws["mask"], None, False, scale, pa, seed(l, 1), step, ws["err"])
            else:
                gm(q, k, ws["scores"], bn=128)
                E.softmax_fwd(ws["scores"], ws["mask"], A["p"], A["pd"] if pa > 0 else None, scale, pa, seed(l, 1), step)
            gm(A["pd"] if pa > 0 else A["p"], v, ctx_view(A["ctx"]), b_mn=True, bn=64)
            gm(A["ctx"], w16[n + "out_w"], ws["tmp"], epi=EPI_BIAS, bias=w32[n + "out_b"])
            E.ln_fwd(ws["tmp"], x, w32[n + "ln1_g"], w32[n + "ln1_b"], A["z1"], A["x1"], A["m1"], A["r1"], eps, ph, seed(l, 2), step)
            gm(A["x1"], w16[n + "w1"], A["u"], epi=EPI_BIAS_GELU, bias=w32[n + "b1"], c2=A["g"])
            gm(A["g"], w16[n + "w2"], ws["tmp"], epi=EPI_BIAS, bias=w32[n + "b2"])
            E.ln_fwd(ws["tmp"], A["x1"], w32[n + "ln2_g"], w32[n + "ln2_b"], A["z2"], A["out"], A["m2"], A["r2"], eps, ph, seed(l, 3), step)
            x = A["out"]
        seq = x
        # next-sentence head
        cls = seq.view(B, S, H)[:, 0]                                                   # [B, H] strided view
        gm(cls, w16["pooler.w"], ws["pooled"], epi=EPI_BIAS_TANH, bias=w32["pooler.b"], bn=128)
        gm(ws["pooled"], w16["nsp.w"], ws["nsp_logits"][:, :2], epi=EPI_BIAS, bias=w32["nsp.b"], bn=64)
        E.xent(ws["nsp_logits"], nsp_labels.reshape(-1), None, ws["one"], ws["loss"], 2, 1.0 / B, False, 0.0)
        # masked-LM head
        torch.add(mlm_positions, torch.arange(B, device=ids.device)[:, None] * S, out=ws["flat_pos"].view(B, P))
        E.gather_rows(seq, ws["flat_pos"], ws["xm"])
        gm(ws["xm"], w16["mlm.dense_w"], ws["hm_u"], epi=EPI_BIAS_GELU, bias=w32["mlm.dense_b"], c2=ws["hm"], bn=128)
        E.ln_fwd(ws["hm"], None, w32["mlm.ln_g"], w32["mlm.ln_b"], None, ws["hl"], ws["mm"], ws["mr"], eps, 0.0, 0, None)
        dec = "emb.word" if c.tie_word_embeddings else "mlm.decoder_w"
        gm(ws["hl"], w16[dec], ws["logits"][:, :V], epi=EPI_BIAS, bias=w32["mlm.bias"])
        E.xent(ws["logits"], mlm_ids.reshape(-1), mlm_weights.reshape(-1).to(torch.float32), ws["denom"], ws["loss"], V, 1.0, True, 1e-5)
        if not backward:
            return ws["loss"]

        # ------------------------------ backward (logits / nsp_logits now hold d loss / d logits)
        ready = self.grad_ready or (lambda lo, hi: None)
        side, use_side = ws["side_stream"], self.side_stream_bias_grads

        def bias_grad(src, dst, slot):
            """dst = column sums of src. On the side stream when enabled: the caller joins before dst or src is needed again."""
            if not use_side:
                E.keyed_colsum(src, None, ws["part"], dst, 1, False)
                return
            ws["side_fork"].record(torch.cuda.current_stream())
            side.wait_event(ws["side_fork"])
            with torch.cuda.stream(side):
                E.keyed_colsum(src, None, ws["side_part"][slot], dst, 1, False)

        def join_side():
            if use_side:
                ws["side_join"].record(side)
                torch.cuda.current_stream().wait_event(ws["side_join"])

        dl = ws["logits"]
        E.keyed_colsum(dl, None, ws["part"], ws["d_bias"], 1, False)
        g["mlm.bias"].copy_(ws["d_bias"][:V])
        dlv = dl[:, :V]
        tied = c.tie_word_embeddings
        if tied:
            g["emb.word"].zero_()
        gm(dlv, ws["hl"], g[dec], a_mn=True, b_mn=True)                               # dE = dlogits^T . hl
        gm(dlv, w16[dec], ws["d_hl"], b_mn=True)                                        # dhl = dlogits . E
        E.ln_bwd(ws["d_hl"], ws["hm"], ws["mm"], ws["mr"], w32["mlm.ln_g"], None, ws["d_hm"], None, ws["ln_part"],
                 g["mlm.ln_g"], g["mlm.ln_b"], 0.0, 0, None, False, None)
        E.gelu_bwd(ws["d_hm"], ws["hm_u"], ws["d_hu"])
        E.keyed_colsum(ws["d_hu"], None, ws["part"], g["mlm.dense_b"], 1, False)
        gm(ws["d_hu"], ws["xm"], g["mlm.dense_w"], a_mn=True, b_mn=True)
        gm(ws["d_hu"], w16["mlm.dense_w"], ws["d_xm"], b_mn=True)
        d_seq = ws["d_a"]
        d_seq.zero_()
        E.scatter_add_rows_bf16(d_seq, ws["flat_pos"], ws["d_xm"])
        # next-sentence head
        dn = ws["nsp_logits"][:, :2]
        g["nsp.b"].copy_(dn.float().sum(0))
        gm(dn, ws["pooled"], g["nsp.w"], a_mn=True, b_mn=True, bn=128)
        gm(dn, w16["nsp.w"], ws["d_pooled"], b_mn=True, bn=128)
        E.tanh_bwd(ws["d_pooled"], ws["pooled"], ws["d_pre"])
        g["pooler.b"].copy_(ws["d_pre"].float().sum(0))
        gm(ws["d_pre"], cls, g["pooler.w"], a_mn=True, b_mn=True, bn=128)
        d_cls = d_seq.view(B, S, H)[:, 0]
        gm(ws["d_pre"], w16["pooler.w"], d_cls, b_mn=True, epi=EPI_ADD, aux=d_cls, bn=128)
        ready(fl.offsets["pooler.w"], fl.total)

        d_out = d_seq
        spare = [ws["d_b"], ws["d_c"]]
        for l in range(c.num_hidden_layers - 1, -1, -1):
            A = ws["layers"][l]
            n = f"layers.{l}."
            x_in = ws["layers"][l - 1]["out"] if l > 0 else ws["x0"]
            dz2, dfo = spare[0], (spare[1] if ph > 0 else spare[0])
            # the layernorm backward also sums what it hands to the linear layer in front of the residual: that layer's bias gradient
            E.ln_bwd(d_out, A["z2"], A["m2"], A["r2"], w32[n + "ln2_g"], None, dz2, dfo if ph > 0 else None, ws["ln_part"],
                     g[n + "ln2_g"], g[n + "ln2_b"], ph, seed(l, 3), step, False, g[n + "b2"])
            gm(dfo, A["g"], g[n + "w2"], a_mn=True, b_mn=True)                          # dW2 = dfo^T . g
            gm(dfo, w16[n + "w2"], ws["d_big"], b_mn=True, epi=EPI_MUL_GELU_GRAD, aux=A["u"])   # dU
            bias_grad(ws["d_big"], g[n + "b1"], 1)
            gm(ws["d_big"], A["x1"], g[n + "w1"], a_mn=True, b_mn=True)                 # dW1 = dU^T . x1
            dx1 = d_out                                                                 # d_out is dead: reuse
            gm(ws["d_big"], w16[n + "w1"], dx1, b_mn=True, epi=EPI_ADD, aux=dz2)        # dx1 = dU . W1 + dz2
            dz1, dao = spare[0], (spare[1] if ph > 0 else spare[0])
            E.ln_bwd(dx1, A["z1"], A["m1"], A["r1"], w32[n + "ln1_g"], None, dz1, dao if ph > 0 else None, ws["ln_part"],
                     g[n + "ln1_g"], g[n + "ln1_b"], ph, seed(l, 2), step, False, g[n + "out_b"])
            gm(dao, A["ctx"], g[n + "out_w"], a_mn=True, b_mn=True)                     # dWo
            dctx = dx1                                                                  # reuse again
            gm(dao, w16[n + "out_w"], dctx, b_mn=True)                                  # dctx = dao . Wo
            q, k, v = (heads_view(A["qkv"], i) for i in range(3))
            dq, dk, dv = (heads_view(ws["d_qkv"], i) for i in range(3))
            pdrop = A["pd"] if pa > 0 else A["p"]
            gm(pdrop, ctx_view(dctx), dv, a_mn=True, b_mn=True, bn=64)                  # dV = P^T . dctx
            if fused_sm:      # dS = scale * P * (dP - sum(dP * P)) in the epilogue of dP = dctx . V^T
                E.gemm_softmax(ctx_view(dctx), v, ws["d_p"], None, None, A["p"], True, scale, pa, seed(l, 1), step, ws["err"])
            else:
                gm(ctx_view(dctx), v, ws["d_p"], bn=128)                                # dP = dctx . V^T
                E.softmax_bwd(ws["d_p"], A["p"], scale, pa, seed(l, 1), step)           # dS (in place)
            gm(ws["d_p"], k, dq, b_mn=True, bn=64)                                      # dQ = dS . K
            gm(ws["d_p"], q, dk, a_mn=True, b_mn=True, bn=64)                           # dK = dS^T . Q
            bias_grad(ws["d_qkv"], g[n + "qkv_b"], 3)
            gm(ws["d_qkv"], x_in, g[n + "qkv_w"], a_mn=True, b_mn=True)                 # dWqkv
            d_prev = dctx
            gm(ws["d_qkv"], w16[n + "qkv_w"], d_prev, b_mn=True, epi=EPI_ADD, aux=dz1)  # dx = dqkv . Wqkv + dz1
            d_out = d_prev           # always ws["d_a"]: the two spare buffers hold this layer's dz / dropped copies
            lo = fl.offsets[n + "qkv_w"]
            hi = fl.offsets[f"layers.{l + 1}.qkv_w"] if l + 1 < c.num_hidden_layers else fl.offsets["pooler.w"]
            join_side()              # the four bias gradients of this layer are complete; their sources may be reused
            ready(lo, hi)
        # embeddings
        dz0 = spare[0]
        E.ln_bwd(d_out, ws["z0"], ws["m0"], ws["r0"], w32["emb.ln_g"], None, dz0, None, ws["ln_part"], g["emb.ln_g"], g["emb.ln_b"],
                 0.0, 0, None, False, None)
        if word_rows is not None:
            word_rows.push(ids, dz0)                   # sparse path: (row ids, rows) go to the shard owners
        else:
            if not tied:
                g["emb.word"].zero_()
            E.scatter_add_rows(g["emb.word"], ids, dz0, 1.0)
        g["emb.pos"].zero_()
        E.strided_rowsum(dz0, g["emb.pos"], S, S, B)
        E.keyed_colsum(dz0, tts, ws["part"], g["emb.tok_type"], c.type_vocab_size, False)
        ready(0, fl.offsets["layers.0.qkv_w"])
        return ws["loss"]


    # ------------------------------------------------------------------ module call
    def forward(self, input_ids, input_mask, segment_ids, mlm_positions, mlm_ids, mlm_weights, nsp_labels):
        if self.flat is not None and input_ids.is_cuda:
            return _FusedBertFn.apply(self, torch.is_grad_enabled(), input_ids, input_mask, segment_ids, mlm_positions,
                                      mlm_ids, mlm_weights, nsp_labels, *self.flat.params[:1])
        return self.reference_loss(input_ids, input_mask, segment_ids, mlm_positions, mlm_ids, mlm_weights, nsp_labels)

    def check_error(self):
        """Raise if a kernel of the last steps reported a bounded wait that gave up."""
        if self._ws is not None:
            code = int(self._ws["err"].item())
            if code:
                what = "an input id lies outside its embedding table" if code == 21 else "a GEMM kernel gave up waiting"
                raise RuntimeError(f"{what} (code {code})")


class _FusedBertFn(torch.autograd.Function):
    """Forward runs the fused forward *and* backward (gradients land in the flat buffer); the autograd backward only
    has to tell autograd that the parameters' ``.grad`` are already in place."""

    @staticmethod
    def forward(ctx, model, train, *args):
        inputs, anchor = args[:7], args[7:]
        loss = model.fused_forward_backward(*inputs, backward=train)
        return loss.clone().view(())

    @staticmethod
    def backward(ctx, grad_out):
        return (None,) * 10


def synthetic_batch(config, batch, seq_len=128, max_predictions=20, seed=0, device="cpu", pin=False):
    """The benchmark's input: uniform token ids, 15 % of positions selected for MLM, uniform NSP labels."""
    g = torch.Generator().manual_seed(seed)
    ids = torch.randint(0, config.vocab_size, (batch, seq_len), generator=g)
    pos = torch.stack([torch.randperm(seq_len, generator=g)[:max_predictions].sort().values for _ in range(batch)])
    out = {
        "input_ids": ids, "input_mask": torch.ones(batch, seq_len, dtype=torch.int64),
        "segment_ids": torch.randint(0, 2, (batch, seq_len), generator=g),
        "mlm_positions": pos, "mlm_ids": torch.gather(ids, 1, pos),
        "mlm_weights": torch.ones(batch, max_predictions, dtype=torch.float32),
        "nsp_labels": torch.randint(0, 2, (batch,), generator=g),
    }
    if pin:
        out = {k: v.pin_memory() for k, v in out.items()}
    return {k: v.to(device) for k, v in out.items()} if device != "cpu" else out
