"""DeepSeek-family forward pass over a packed ragged batch with a paged latent-KV pool.

Two implementations of the same math:

* `forward_reference` - plain PyTorch (fp32 math on bf16-rounded activations at the same
  boundaries as the kernels).  Runs anywhere; it is the CPU execution path and the oracle.
* `forward_cuda`      - the sm_100a kernel pipeline (tcgen05 GEMMs, MLA attention, fused
  small ops), allocation-free over a preallocated workspace so a decode step can be
  captured in a CUDA graph.

Layer structure (weight-absorbed MLA, pre-norm residual):
  h -> RMSNorm -> [q | c_kv,k_rope] -> (q_norm, q_b) -> RoPE, KV append -> q_nope @ W_UK
    -> paged attention over latent rows -> @ W_UV -> o_proj (+ all-reduce) -> + h
    -> RMSNorm -> dense SwiGLU FFN | router -> top-k -> grouped experts (+ shared) -> + h

Layer-level counterpart of crates/ferrule-model/src/models/deepseek_v4/layer.rs:391-470 and
attention.rs:1194-1364 in the reference (whose V4-only extras live in `v4.py`).
"""
from __future__ import annotations

from dataclasses import dataclass
from typing import Optional

import torch

from ..ops import reference as ref
from .config import ModelConfig
from .weights import LayerWeights, ModelWeights, QuantWeight


@dataclass
class DeviceBatch:
    """Device-side view of one packed execution batch (all tensors on the model's device).

    rows may exceed n_rows (padding up to a graph bucket): padded rows carry write_slot = -1
    and row_pos = -1 and never touch the KV pool.
    """
    token_ids: torch.Tensor     # [rows] int32
    positions: torch.Tensor     # [rows] int32 absolute position of each token
    write_slot: torch.Tensor    # [rows] int64 pool row the token's KV is written to (-1: none)
    row_seq: torch.Tensor       # [rows] int32 index into block_table
    row_pos: torch.Tensor       # [rows] int32 last KV position visible to the row (= position)
    block_table: torch.Tensor   # [seqs, max_blocks] int32 page ids
    logit_rows: torch.Tensor    # [n_logit] int32 rows whose logits are wanted
    n_rows: int
    n_logit: int
    decode_only: bool = False   # every sequence has exactly one row (a plain decode step)
    tc_tiles: Optional[torch.Tensor] = None     # [cap, 4] int32 tiles of the tensor-core prefill attention kernel
    n_tc_tiles: int = 0
    rest_ranges: Optional[list] = None          # (first row, end row) ranges the tiles do not cover


class KvPool:
    """Physical paged latent-KV pool: [layers, pages, page_size, kv_lora + rope] bf16 (fp32 on CPU)."""

    def __init__(self, cfg: ModelConfig, n_pages: int, page_size: int, device, dtype=torch.bfloat16,
                 n_layers: Optional[int] = None):
        self.cfg, self.n_pages, self.page_size = cfg, n_pages, page_size
        self.n_layers = cfg.n_layers + cfg.n_mtp_layers if n_layers is None else n_layers
        self.data = torch.zeros(self.n_layers, n_pages, page_size, cfg.kv_row_dim, dtype=dtype, device=device)

    def layer(self, i: int) -> torch.Tensor:
        return self.data[i]

    @property
    def bytes_per_page(self) -> int:
        return self.n_layers * self.page_size * self.cfg.kv_row_dim * self.data.element_size()

    def copy_pages(self, pairs) -> None:
        """Copy whole pages (all layers): pairs = [(src, dst), ...] (copy-on-write)."""
        if not pairs:
            return
        if self.data.is_cuda:
            from ..ops import kernels as K
            K.copy_pages(self.data, torch.tensor(pairs, dtype=torch.int32, device=self.data.device))
        else:
            for s, d in pairs:
                self.data[:, d] = self.data[:, s]

    def snapshot_pages(self, pages) -> torch.Tensor:
        """Device -> host copy of pages (session preemption)."""
        idx = torch.tensor(list(pages), dtype=torch.long, device=self.data.device)
        return self.data[:, idx].to("cpu", copy=True)

    def restore_pages(self, pages, snap: torch.Tensor) -> None:
        idx = torch.tensor(list(pages), dtype=torch.long, device=self.data.device)
        self.data[:, idx] = snap.to(self.data.device)


# ======================================================================================
# reference forward (PyTorch)
# ======================================================================================
class ReferenceForward:
    """fp32 PyTorch implementation; `emulate_bf16` rounds activations where the kernels do."""

    def __init__(self, weights: ModelWeights, pool: KvPool, emulate_bf16: bool = False):
        self.w, self.cfg, self.pool = weights, weights.cfg, pool
        self.rnd = ref.bf16_round if emulate_bf16 else (lambda t: t)
        self.expert_gate = None        # callable(layer, local experts) used by the asynchronous expert streaming
        self.route_observer = None     # callable(layer, expert ids [T, k], T): route statistics (parallel/placement.py)
        self.prof = None               # utils.stage_profile.StageProfiler: per-layer stage table
        self.tap = None                # utils.stage_profile.DebugTap: dumps of intermediate rows
        # sequence parallelism (parallel.tp.TensorParallel with the host collectives): between the reduce-scatter
        # after a sublayer and the all-gather in front of the next one every rank holds only its slice of the rows -
        # residual stream, residual adds and norms are sharded by rows, the collectives move the same bytes as the
        # all-reduce they replace
        self.sp = None
        self._layer_index = -1
        cfg = self.cfg
        dev = weights.embed.device
        cos, sin = ref.rope_tables(min(cfg.max_position, 1 << 16), cfg.qk_rope_dim, cfg.rope_theta,
                                   cfg.rope_factor, cfg.rope_orig_max_pos, cfg.rope_beta_fast,
                                   cfg.rope_beta_slow)
        self.cos, self.sin = cos.to(dev), sin.to(dev)
        # oracle of an FP8 model: inputs of quantised linears go through the 1 x 128 FP8 round trip
        if getattr(weights, "act_quant", False):
            from ..io import encoding as enc
            db = getattr(weights, "dense_act_block", 128)
            self.aq = lambda x: enc.act_dequant_fp8(*enc.act_quant_fp8(x, db), db)
            eb = getattr(weights, "expert_act_block", 128)
            self.aq_e = lambda x: enc.act_dequant_fp8(*enc.act_quant_fp8(x, eb), eb)
        else:
            self.aq = self.aq_e = lambda x: x

    # -- pieces ------------------------------------------------------------------------
    def _attention(self, lw: LayerWeights, layer: int, xn: torch.Tensor, b: DeviceBatch) -> torch.Tensor:
        cfg, rnd = self.cfg, self.rnd
        xn = self.aq(xn)
        T = xn.shape[0]
        hl = self.w.heads_local
        qhd, lora, rope, nope = cfg.q_head_dim, cfg.kv_lora_rank, cfg.qk_rope_dim, cfg.qk_nope_dim
        qkv = rnd(xn @ lw.w_qkv_a.float().T)
        if cfg.q_lora_rank:
            qa, ckv = qkv[:, :cfg.q_lora_rank], qkv[:, cfg.q_lora_rank:]
            qn = rnd(ref.rmsnorm(qa, lw.q_norm, cfg.rms_eps))
            q = rnd(self.aq(qn) @ lw.w_q_b.float().T)
        else:
            q, ckv = qkv[:, :hl * qhd], qkv[:, hl * qhd:]
        q = q.view(T, hl, qhd)
        pos = b.positions[:T].long()
        c, s = self.cos[pos], self.sin[pos]
        q_rope = rnd(ref.apply_rope(q[:, :, nope:], c[:, None], s[:, None]))
        kv_lat = rnd(ref.rmsnorm(ckv[:, :lora], lw.kv_norm, cfg.rms_eps))
        k_rope = rnd(ref.apply_rope(ckv[:, lora:], c, s))
        kv_row = torch.cat([kv_lat, k_rope], dim=-1)
        pool_l = self.pool.layer(layer).view(-1, cfg.kv_row_dim)
        slots = b.write_slot[:T]
        ok = slots >= 0
        pool_l[slots[ok]] = kv_row[ok].to(pool_l.dtype)
        q_lat = rnd(torch.einsum("thk,hnk->thn", q[:, :, :nope], lw.w_uk_t.float()))
        q_full = torch.cat([q_lat, q_rope], dim=-1)
        o_lat = rnd(ref.mla_paged_attention(q_full, pool_l, b.block_table, b.row_seq[:T], b.row_pos[:T],
                                            self.pool.page_size, lora, cfg.softmax_scale, sink=lw.attn_sink))
        o = rnd(torch.einsum("thk,hnk->thn", o_lat, lw.w_uv.float())).reshape(T, -1)
        return self.aq(o) @ lw.w_o.float().T          # partial sum over this rank's heads

    def _ffn(self, w13: torch.Tensor, w2: torch.Tensor, x: torch.Tensor) -> torch.Tensor:
        inter = w13.shape[-2] // 2
        y = self.aq(x) @ w13[0].float().T
        h = self.rnd(ref.swiglu(y[:, :inter], y[:, inter:], self.cfg.swiglu_limit))
        return self.aq(h) @ w2[0].float().T

    def _moe(self, lw: LayerWeights, xn: torch.Tensor, token_ids: torch.Tensor) -> torch.Tensor:
        cfg, rnd = self.cfg, self.rnd
        logits = xn @ lw.router_w.float().T
        idx, wts = ref.route(logits, cfg.topk, cfg.score_fn, bias=lw.router_bias, n_groups=cfg.n_groups,
                             topk_groups=cfg.topk_groups, normalize=cfg.norm_topk_prob,
                             route_scale=cfg.route_scale, hash_table=lw.hash_table, token_ids=token_ids)
        I = cfg.moe_inter
        out = torch.zeros_like(xn)
        if self.route_observer is not None:
            self.route_observer(self._layer_index, idx, xn.shape[0])
        if self.expert_gate is not None:
            # streamed experts: the gate raises when the batch routes to experts that are not resident
            local = idx[(idx >= self.w.e_lo) & (idx < self.w.e_hi)] - self.w.e_lo
            self.expert_gate(self._layer_index, sorted(set(local.flatten().tolist())))
        for e in range(self.w.e_lo, self.w.e_hi):
            hit = (idx == e)
            rows = hit.any(-1).nonzero().flatten()
            if rows.numel() == 0:
                continue
            wsel = (wts * hit)[rows].sum(-1, keepdim=True)
            y = self.aq_e(xn[rows]) @ lw.e_w13[e - self.w.e_lo].float().T
            h = rnd(ref.swiglu(y[:, :I], y[:, I:], cfg.swiglu_limit))
            out[rows] += rnd((self.aq_e(h) @ lw.e_w2[e - self.w.e_lo].float().T) * wsel)
        if lw.w13 is not None:
            out = out + rnd(self._ffn(lw.w13, lw.w2, xn))
        return out

    def layer_sp(self, lw: LayerWeights, layer: int, h_rows: torch.Tensor, b: DeviceBatch, T: int) -> torch.Tensor:
        """One layer on row-sharded activations: `h_rows` are this rank's rows of the residual stream (in and out).
        all-gather(norm(rows)) -> sublayer on all rows with this rank's heads / experts -> reduce-scatter -> add."""
        cfg, rnd, sp = self.cfg, self.rnd, self.sp
        self._layer_index = layer
        xn = sp.all_gather_reference(rnd(ref.rmsnorm(h_rows, lw.attn_norm, cfg.rms_eps)), T)
        a = self._attention(lw, layer, xn, b)
        h_rows = rnd(h_rows + sp.reduce_scatter_reference(a.contiguous()))
        xn = sp.all_gather_reference(rnd(ref.rmsnorm(h_rows, lw.ffn_norm, cfg.rms_eps)), T)
        f = self._moe(lw, xn, b.token_ids[:T]) if lw.is_moe else self._ffn(lw.w13, lw.w2, xn)
        return rnd(h_rows + sp.reduce_scatter_reference(f.contiguous()))

    def layer(self, lw: LayerWeights, layer: int, h: torch.Tensor, b: DeviceBatch, allreduce=None) -> torch.Tensor:
        cfg, rnd = self.cfg, self.rnd
        T = h.shape[0]
        self._layer_index = layer
        prof, tap = self.prof, self.tap
        if prof is not None:
            prof.mark(layer, "attn")
        xn = rnd(ref.rmsnorm(h, lw.attn_norm, cfg.rms_eps))
        a = self._attention(lw, layer, xn, b)
        if prof is not None:
            prof.mark(layer, "attn.reduce")
        if allreduce is not None:
            a = allreduce(a)
        else:
            a = rnd(a)
        h = rnd(h + a)
        if tap is not None:
            tap.write(layer, "attn_out", h)
        if prof is not None:
            prof.mark(layer, "moe" if lw.is_moe else "ffn")
        xn = rnd(ref.rmsnorm(h, lw.ffn_norm, cfg.rms_eps))
        f = self._moe(lw, xn, b.token_ids[:T]) if lw.is_moe else self._ffn(lw.w13, lw.w2, xn)
        if prof is not None:
            prof.mark(layer, "ffn.reduce")
        if allreduce is not None:
            f = allreduce(f)
        elif not lw.is_moe:
            f = rnd(f)
        out = rnd(h + f)
        if prof is not None:
            prof.mark(layer, None)
        if tap is not None:
            tap.write(layer, "layer_out", out)
        return out

    def embed_rows(self, b: DeviceBatch) -> torch.Tensor:
        return self.w.embed[b.token_ids[:b.n_rows].long()].float()

    def run_layers(self, h: torch.Tensor, b: DeviceBatch, allreduce=None, start_layer: int = 0) -> torch.Tensor:
        """The layers this weight image holds (all of them, or one pipeline stage's share), from `start_layer`
        (a resumed transaction continues at the layer it stopped at, with that layer's input rows as `h`)."""
        if self.sp is not None and allreduce is not None and self.sp.world > 1:
            # sequence parallel: every rank enters with the replicated rows, keeps its slice through the layers and
            # gathers the slices once at the end
            T = h.shape[0]
            lo, hi = self.sp.row_range(T)
            rows = h[lo:hi].contiguous()
            for i, lw in enumerate(self.w.layers):
                if i >= start_layer:
                    rows = self.layer_sp(lw, i, rows, b, T)
            return self.sp.all_gather_reference(rows, T)
        for i, lw in enumerate(self.w.layers):
            if i < start_layer:
                continue
            try:
                h = self.layer(lw, i, h, b, allreduce)
            except Exception as exc:  # noqa: BLE001
                if hasattr(exc, "missing"):
                    exc.hidden = h
                raise
        return h

    def hidden_states(self, b: DeviceBatch, allreduce=None, start_layer: int = 0, h0=None) -> torch.Tensor:
        h = self.embed_rows(b) if h0 is None else h0
        return self.run_layers(h, b, allreduce, start_layer)

    def logits_from_hidden(self, h: torch.Tensor, b: DeviceBatch, final_norm=None, lm_head=None) -> torch.Tensor:
        rows = b.logit_rows[:b.n_logit].long()
        hn = self.rnd(ref.rmsnorm(h[rows], self.w.final_norm if final_norm is None else final_norm,
                                  self.cfg.rms_eps))
        return hn @ (self.w.lm_head if lm_head is None else lm_head).float().T

    def forward(self, b: DeviceBatch, allreduce=None, gather_vocab=None, return_hidden: bool = False):
        """-> fp32 logits [n_logit, vocab_local] (or gathered vocab with `gather_vocab`)."""
        h = self.hidden_states(b, allreduce)
        logits = self.logits_from_hidden(h, b)
        if gather_vocab is not None:
            logits = gather_vocab(logits)
        return (logits, h) if return_hidden else logits

    def mtp_forward(self, stage: int, h_prev: torch.Tensor, b: DeviceBatch, allreduce=None):
        """One MTP stage: rows carry the *next* token ids; h_prev are the main-model hidden states
        of the same rows.  Returns (logits over logit_rows, hidden)."""
        m = self.w.mtp[stage]
        cfg, rnd = self.cfg, self.rnd
        T = b.n_rows
        e = (self.w.embed if m.embed is None else m.embed)[b.token_ids[:T].long()].float()
        # column order of eh_proj in published DeepSeek-V3 checkpoints: [enorm(embedding) ; hnorm(previous hidden)]
        x = torch.cat([rnd(ref.rmsnorm(e, m.enorm, cfg.rms_eps)), rnd(ref.rmsnorm(h_prev, m.hnorm, cfg.rms_eps))], -1)
        h = rnd(x @ m.eh_proj.float().T)
        h = self.layer(m.layer, cfg.n_layers + stage, h, b, allreduce)
        return self.logits_from_hidden(h, b, final_norm=m.final_norm, lm_head=m.lm_head), h


# ======================================================================================
# CUDA forward (sm_100a kernels)
# ======================================================================================
def _pow2_at_least(x: float, lo: int, hi: int) -> int:
    n = lo
    while n < x and n < hi:
        n *= 2
    return n


class CudaWorkspace:
    """Preallocated activations for up to `max_rows` packed rows (no allocation while stepping)."""

    def __init__(self, w: ModelWeights, max_rows: int, max_logit_rows: int, decode_rows: int,
                 attn_splits: int, device):
        cfg = w.cfg
        hl = w.heads_local
        H, D = cfg.hidden, cfg.kv_row_dim
        bf = dict(dtype=torch.bfloat16, device=device)
        f32 = dict(dtype=torch.float32, device=device)
        i32 = dict(dtype=torch.int32, device=device)
        R = max_rows
        self.max_rows, self.max_logit_rows = R, max_logit_rows
        self.h = [torch.zeros(R, H, **bf), torch.zeros(R, H, **bf)]
        self.xn = torch.zeros(R, H, **bf)
        self.qkv = torch.zeros(R, w.layers[0].w_qkv_a.shape[0], **bf)
        self.q = torch.zeros(R, hl * cfg.q_head_dim, **bf) if cfg.q_lora_rank else None
        self.qn = torch.zeros(R, cfg.q_lora_rank, **bf) if cfg.q_lora_rank else None
        self.q_full = torch.zeros(R, hl, D, **bf)
        # decode on folded weights, models without a query down-projection: one GEMM writes q_full's layout and the
        # latent-kv row side by side
        self.q_fold = None if cfg.q_lora_rank else torch.zeros(min(R, 4 * decode_rows), (hl + 1) * D, **bf)
        self.o_lat = torch.zeros(R, hl, cfg.kv_lora_rank, **bf)
        self.attn_out = torch.zeros(R, hl * cfg.v_head_dim, **bf)
        self.delta = torch.zeros(R, H, **bf)
        inter_max = 0
        for lw in list(w.layers) + [m.layer for m in w.mtp]:
            if lw.w13 is not None:
                inter_max = max(inter_max, lw.w13.shape[1] // 2)
        self.ffn_mid = torch.zeros(R, max(inter_max, 8), **bf)
        self.attn_splits = attn_splits
        self.decode_rows = decode_rows
        from ..ops.kernels import AttnWorkspace, MoePlan
        sr = 4 * decode_rows        # split attention also serves verification batches (see _attention)
        self.attn_ws = AttnWorkspace(torch.zeros(sr, attn_splits, hl, cfg.kv_lora_rank, **f32),
                                     torch.zeros(sr, attn_splits, hl, 2, **f32), sr, attn_splits,
                                     torch.zeros(sr * ((hl + 15) // 16), **i32)) \
            if attn_splits > 1 and attn_splits not in (2, 4, 8) else None
        self.has_moe = cfg.n_routed_experts > 0
        self.router_ctr = torch.zeros(4, **i32)
        from ..ops.kernels import ArgmaxScratch
        self.argmax_scratch = ArgmaxScratch.allocate(max(max_logit_rows, 1), device)
        if self.has_moe:
            E, k = cfg.n_routed_experts, cfg.topk
            el = w.e_hi - w.e_lo
            self.router_logits = torch.zeros(R, E, **f32)
            self.topk_idx = torch.zeros(R, k, **i32)
            self.topk_w = torch.zeros(R, k, **f32)
            self.slots = k + 1
            self.plans = {}
            for ntok in (16, 32, 64, 128):
                self.plans[ntok] = MoePlan.allocate(R * k, el, ntok, device)
            # expert-major rows: routes of the largest batch, or the static decode layout (64 rows per local expert)
            xrows = max(R * k, el * 64)
            self.xg = torch.zeros(xrows, H, **bf)
            self.hmid = torch.zeros(xrows, cfg.moe_inter, **bf)
            # decode-sized batches: one fixed row tile per local expert, row counters per layer zeroed once a step
            from ..ops.kernels import static_plan
            n_slots = cfg.n_layers + len(w.mtp)
            self.route_cnt = torch.zeros(n_slots, el, **i32)
            self.static_rows = [16, 32, 64]
            self.static_plans = {}
            for nt in self.static_rows:
                base = static_plan(nt, el, self.route_cnt[0])
                self.static_plans[nt] = [base] + [static_plan(nt, el, self.route_cnt[j], base)
                                                  for j in range(1, n_slots)]
            self.route_out = torch.zeros(R, self.slots, H, **bf)
        L = max_logit_rows
        self.h_last = torch.zeros(L, H, **bf)
        self.hn_last = torch.zeros(L, H, **bf)
        self.logits = torch.zeros(L, w.lm_head.shape[0], **f32)
        # greedy result packed for a single device->host copy: [ids (int32) | values (fp32 bits)]
        self.out_buf = torch.zeros(2 * L, **i32)
        self.next_id = self.out_buf[:L]
        self.next_val = self.out_buf[L:].view(torch.float32)
        self.mtp_x = torch.zeros(R, 2 * H, **bf) if w.mtp else None
        # FP8 models: e4m3 codes + UE8M0 scales (one per 1 x 128) of the activation rows feeding each linear
        self.act_q = {}
        if w.weight_format != "bf16":
            u8 = dict(dtype=torch.uint8, device=device)

            def pair(rows, width):
                width = (max(width, 128) + 127) // 128 * 128
                return torch.zeros(rows, width, **u8), torch.zeros(rows, width // 128, **u8)

            self.act_q["xn"] = pair(R, H)
            self.act_q["a"] = pair(R, max(cfg.q_lora_rank, hl * cfg.v_head_dim, 2 * H if w.mtp else 0))
            self.act_q["mid"] = pair(R, inter_max)
            if self.has_moe:
                qrows = max(R * cfg.topk, (w.e_hi - w.e_lo) * 64)       # routes, or the static decode slots
                self.act_q["xg"] = pair(qrows, H)
                self.act_q["hmid"] = pair(qrows, cfg.moe_inter)
            all_layers = list(w.layers) + [m.layer for m in w.mtp]
            if any(isinstance(v, QuantWeight) and v.native_mx for l in all_layers if l is not None
                   for v in vars(l).values()):
                # MXFP8 activations (codes + one scale byte per 1 x 32 block) of the linears whose weights run on
                # the block-scaled tensor-core GEMM: natively held MXFP4 experts, FP8 weights with replicated scales
                def pair32(rows, width):
                    width = (max(width, 128) + 127) // 128 * 128
                    return torch.zeros(rows, width, **u8), torch.zeros(rows, width // 32, **u8)
                self.act_q["xn_mx"] = pair32(R, H)
                self.act_q["a_mx"] = pair32(R, self.act_q["a"][0].shape[1])
                self.act_q["mid_mx"] = pair32(R, inter_max)
                if self.has_moe:
                    xrows = max(R * cfg.topk, (w.e_hi - w.e_lo) * 64)
                    self.act_q["xg_mx"] = pair32(xrows, H)
                    self.act_q["hmid_mx"] = pair32(xrows, cfg.moe_inter)

    def nbytes(self) -> int:
        tot = 0
        for v in vars(self).values():
            ts = v if isinstance(v, (list, tuple)) else [v]
            for t in ts:
                if isinstance(t, torch.Tensor):
                    tot += t.numel() * t.element_size()
        return tot


def cfg_inter_bad(cfg) -> bool:
    """The quantised SwiGLU output needs whole 128-channel scale blocks."""
    return cfg.moe_inter % 128 != 0 or cfg.hidden % 128 != 0


class CudaForward:
    """The kernel pipeline.  `tp` (parallel.tp.TensorParallel) supplies the fused collectives;
    None means a single GPU."""

    def __init__(self, weights: ModelWeights, pool: KvPool, max_rows: int = 4096,
                 max_logit_rows: int = 256, decode_rows: int = 64, max_seq_len: int = 4096,
                 attn_splits: int = 8, tp=None):
        from ..ops import kernels as K
        from ..ops import movers as M
        from ..ops import quant as Q
        self.K, self.Q, self.M = K, Q, M
        self.w, self.cfg, self.pool, self.tp = weights, weights.cfg, pool, tp
        dev = weights.embed.device
        self.device = dev
        cfg = self.cfg
        import os
        attn_splits = int(os.environ.get("FERRULE_ATTN_SPLITS", attn_splits))
        # FP8 models: activation quantisation in the producing kernels (norm -> FP8, SwiGLU -> FP8) instead of
        # one quantiser launch per consumer
        self.fuse_act_quant = os.environ.get("FERRULE_FUSE_ACT_QUANT", "1") != "0"
        self.fp8_static = os.environ.get("FERRULE_FP8_STATIC", "1") != "0"
        # rows per tile when the block-scaled GEMM walks a static slot (0: one tile per slot).  Measured on the
        # V2-Lite shape: 16-row sub-tiles lose (5.67 vs 5.21 ms per step in FP8: twice the work items, half of them
        # skipped) and change nothing on the V3 shard, so one tile per slot is the default.
        self.mx_slot_ntok = int(os.environ.get("FERRULE_MX_SLOT_NTOK", "0"))
        self._quantised = {}        # act_q slot -> (source pointer, rows, width) whose FP8 form the slot holds
        self.max_seq_len = max_seq_len
        self.split_tokens = max(64, ((max_seq_len + attn_splits - 1) // attn_splits + 63) // 64 * 64)
        self.ws = CudaWorkspace(weights, max_rows, max_logit_rows, decode_rows, attn_splits, dev)
        cos, sin = ref.rope_tables(min(cfg.max_position, max(max_seq_len, 16)), cfg.qk_rope_dim, cfg.rope_theta,
                                   cfg.rope_factor, cfg.rope_orig_max_pos, cfg.rope_beta_fast, cfg.rope_beta_slow)
        self.cos, self.sin = cos.to(dev).contiguous(), sin.to(dev).contiguous()
        self.launches = 0          # kernels launched by the last forward (for reporting)
        self.fused_router_rows = 256
        self.side_stream = torch.cuda.Stream(device=dev)      # shared experts run beside the routed path
        self.arena = None          # models.expert_arena.ExpertArena when routed experts are streamed
        self.wave_state = None     # per-transaction {layer: finished waves + their rows} of the asynchronous streaming
        # bytes of each MoE layer's routed-expert weights to prefetch into L2 during the attention half of a decode
        # layer (0 = off); the L2 holds 126 MB, the prefetch must leave room for the attention's own traffic
        import os
        # measured on one GPU with evict-first weight streaming: 0 / 32 / 64 / 96 MB -> 7.38 / 7.33 / 7.29 / 7.55 ms,
        # but once the cache-write kernel runs as a parallel branch the extra branch costs more than it hides
        # (6.75 ms without, 6.97 ms with 48 MB): off by default
        self.l2_prefetch_bytes = int(float(os.environ.get("FERRULE_L2_PREFETCH_MB", "0")) * (1 << 20))
        self.telemetry = None      # utils.telemetry.ExpertTelemetry fed by the streamed path
        self.predictor = None      # runtime.expert_prediction.ExpertPredictor fed by the streamed path
        # callable(layer, expert ids [T, k] on the device, T): route statistics for placement planning.  The observer
        # reads the ids on the host, so a forward that has one is neither captured in a graph nor overlapped
        self.route_observer = None
        # sequence parallelism for batches above the fused all-reduce's row limit (bf16 weights, replicated-activation
        # MoE): the residual stream stays sharded by rows between a sublayer's reduce-scatter and the next all-gather
        self.sequence_parallel = False
        # utils.stage_profile: per-layer stage table (marks are CUDA events on the launching stream; a profiled
        # forward is not captured in a graph) and dumps of intermediate rows
        self.prof = None
        self.tap = None
        self.static_moe = os.environ.get("FERRULE_STATIC_MOE", "1") != "0"
        self.fuse_next_norm = os.environ.get("FERRULE_FUSE_NORM", "1") != "0"
        # measured: folding the post-attention add + RMSNorm into the router kernel loses 10 us per layer, because the
        # shared-expert branch can then only fork after the router instead of running beside it; opt-in
        self.fuse_router_norm = os.environ.get("FERRULE_FUSE_ROUTER_NORM", "0") == "1"
        # measured: prefetching the next layer's attention weights during the MoE phase costs 0.7 ms per step
        # (7.05 -> 7.78 ms): the branch delays the shared-expert join; opt-in only
        self.attn_prefetch = os.environ.get("FERRULE_ATTN_PREFETCH", "0") == "1"
        self._prefetch_next = None
        self.fork_prep = os.environ.get("FERRULE_FORK_PREP", "1") != "0"
        self.prep_stream = torch.cuda.Stream(device=dev)
        # Decode-sized batches can run attention on folded weights: W_UK multiplied into the query projection and W_UV
        # into the output projection, so the two small per-head GEMMs (and their launches) leave the layer.  The folded
        # matrices are 2.5x / 4x larger, and that costs more than the two launches save.  Measured, full
        # DeepSeek-V2-Lite decode step, batch 64: 6.55 -> 7.03 ms whole model, 3.37 -> 3.58 ms on a 4-way head shard,
        # 2.87 -> 2.91 ms on an 8-way shard.  Opt-in ("1"); "auto" folds from 16-way head shards on.  bf16 weights only.
        self.fold_decode = os.environ.get("FERRULE_FOLD_DECODE", "0")
        self._folded = {}
        self.async_stream = False  # streamed experts: stop at a layer with missing experts instead of uploading inline
        # token-dispatch expert parallelism (parallel.ep.ExpertParallelMoE): MoE layers run on this rank's slice of
        # the batch's tokens, routes travel to the experts' owners and back, the slices are gathered for the next layer
        self.ep = None
        self.lease_sink = None     # dict layer -> leases of the running transaction (set by the runner)
        if self._fold_wanted():
            for i, lw in enumerate(self.w.layers):
                self._folded[i] = self._build_fold(lw)

    # -- sublayers -----------------------------------------------------------------------
    # -- linear dispatch -------------------------------------------------------------------
    def _quant(self, x: torch.Tensor, slot: str):
        """1 x 128 FP8 quantisation of activation rows into the workspace pair named `slot`."""
        q, s = self.ws.act_q[slot]
        rows, n = x.shape
        q, s = q[:rows, :n], s[:rows, :n // 128]
        done = self._quantised.get(slot)
        if done is not None and done == (x.data_ptr(), rows, n):
            return q, s                     # the kernel that produced `x` wrote its FP8 form as well
        self.Q.quant_fp8_rows(x, out=(q, s))
        return q, s

    def _quant_mx(self, x: torch.Tensor, slot: str):
        """1 x 32 MXFP8 quantisation of activation rows into the workspace pair named `slot`."""
        q, s = self.ws.act_q[slot]
        rows, n = x.shape
        q, s = q[:rows, :n], s[:rows, :n // 32]
        done = self._quantised.get(slot)
        if done is not None and done == (x.data_ptr(), rows, n):
            return q, s                     # the kernel that produced `x` wrote its MXFP8 form as well
        self.Q.quant_mxfp8_rows(x, out=(q, s))
        return q, s

    @staticmethod
    def _qkind(w) -> Optional[str]:
        """How the rows feeding linear `w` are quantised: 'mx' (1 x 32, block-scaled tensor-core GEMM), 'fp8'
        (1 x 128, FP8 GEMM that rescales k-blocks in its epilogue), None (bf16 weights or MXFP4 in containers)."""
        if not isinstance(w, QuantWeight):
            return None
        if w.native_mx:
            return "mx"
        return None if w.group32 else "fp8"

    def _norm(self, x, weight, T: int, out: torch.Tensor, slot: Optional[str], kind: Optional[str], **kw):
        """add + RMSNorm into `out`; with `kind` (how the consuming linears take their rows, see `_qkind`) the
        kernel also writes the rows' quantised form into the workspace pair of `slot`, and quantising `out` for
        that slot becomes a no-op until the slot's source is rewritten."""
        n = out.shape[1]
        for k_ in (slot, None if slot is None else slot + "_mx"):
            if k_ is not None:
                self._quantised.pop(k_, None)
        if kind is not None and slot is not None and self.fuse_act_quant and n % 128 == 0:
            key = slot + "_mx" if kind == "mx" else slot
            blk = 32 if kind == "mx" else 128
            q, s = self.ws.act_q[key]
            self.K.add_rmsnorm(x, weight, self.cfg.rms_eps, norm_out=out, quant_out=(q[:T, :n], s[:T, :n // blk]),
                               quant_block=blk, **kw)
            self._quantised[key] = (out.data_ptr(), T, n)
        else:
            self.K.add_rmsnorm(x, weight, self.cfg.rms_eps, norm_out=out, **kw)

    def _gemm(self, x, w, out, slot: str = "a", xq=None, **kw):
        """bf16 weight -> bf16 tcgen05 GEMM; QuantWeight -> quantise the rows (unless `xq` is given) and run the
        block-scaled GEMM its form takes.  `q_slot`: the consumer of `out` is a linear of the same form - leave
        the result quantised in that workspace pair (the bf16 `out` is then not written) when the shape allows."""
        q_slot = kw.pop("q_slot", None)
        for k_ in (q_slot, None if q_slot is None else q_slot + "_mx"):
            if k_ is not None:
                self._quantised.pop(k_, None)
        if isinstance(w, QuantWeight) and w.native_mx:
            if xq is None:
                xq = self._quant_mx(x, slot + "_mx")
            codes, fp8 = (w.q, True) if w.packed is None else (w.packed, False)
            if q_slot is not None and self.fuse_act_quant and out.shape[1] % 32 == 0:
                rows, n = out.shape
                oq, os_ = self.ws.act_q[q_slot + "_mx"]
                self.Q.gemm_mxfp4(xq[0], xq[1], codes, w.sf, out_mx=(oq[:rows, :n], os_[:rows, :n // 32]), w_fp8=fp8, **kw)
                self._quantised[q_slot + "_mx"] = (out.data_ptr(), rows, n)
                return out
            return self.Q.gemm_mxfp4(xq[0], xq[1], codes, w.sf, out=out, w_fp8=fp8, **kw)
        if isinstance(w, QuantWeight):
            if xq is None:
                xq = self._quant(x, slot)
            if q_slot is not None:
                rows, n = out.shape
                if self.fuse_act_quant and not w.group32 and n % 128 == 0:
                    oq, os_ = self.ws.act_q[q_slot]
                    self.Q.gemm_fp8(xq[0], xq[1], w.q, w.scale, out_q=(oq[:rows, :n], os_[:rows, :n // 128]), **kw)
                    self._quantised[q_slot] = (out.data_ptr(), rows, n)
                    return out
            return self.Q.gemm_fp8(xq[0], xq[1], w.q, w.scale, out=out, group32=w.group32, **kw)
        return self.K.gemm(x, w, out=out, **kw)

    def _attention(self, lw: LayerWeights, layer: int, xn: torch.Tensor, b: DeviceBatch, T: int) -> torch.Tensor:
        K, cfg, ws = self.K, self.cfg, self.ws
        hl = self.w.heads_local
        qhd, lora, rope, nope, vd = cfg.q_head_dim, cfg.kv_lora_rank, cfg.qk_rope_dim, cfg.qk_nope_dim, cfg.v_head_dim
        fold = self._folded.get(layer) if (T <= 4 * ws.decode_rows and not b.n_tc_tiles) else None
        if fold is not None:
            return self._attention_folded(lw, fold, layer, xn, b, T)
        prof = self.prof
        if prof is not None:
            prof.mark(layer, "attn.qkv")
        qkv = ws.qkv[:T]
        self._gemm(xn, lw.w_qkv_a, qkv, slot="xn")
        if cfg.q_lora_rank:
            qa, ckv = qkv[:, :cfg.q_lora_rank], qkv[:, cfg.q_lora_rank:]
            self._norm(qa, lw.q_norm, T, ws.qn[:T], "a", self._qkind(lw.w_q_b))
            q = self._gemm(ws.qn[:T], lw.w_q_b, ws.q[:T], slot="a")
            self._quantised.pop("a", None)          # the slot is reused for the attention output below
            self._quantised.pop("a_mx", None)
        else:
            q, ckv = qkv[:, :hl * qhd], qkv[:, hl * qhd:]
        if prof is not None:
            prof.mark(layer, "attn.prep+absorb")
        q_full = ws.q_full[:T]
        # the cache write / RoPE kernel and the W_UK absorption GEMM both only read q (they fill disjoint columns
        # of q_full): decode-sized batches run them as parallel branches
        fork = self.fork_prep and T <= ws.decode_rows
        if fork:
            main = torch.cuda.current_stream()
            self.prep_stream.wait_stream(main)
            with torch.cuda.stream(self.prep_stream):
                K.mla_prep(q, qhd, ckv, hl, lora, rope, lw.kv_norm, cfg.rms_eps, self.cos, self.sin,
                           b.positions, b.write_slot, self.pool.layer(layer), q_full.view(T, -1))
        else:
            K.mla_prep(q, qhd, ckv, hl, lora, rope, lw.kv_norm, cfg.rms_eps, self.cos, self.sin,
                       b.positions, b.write_slot, self.pool.layer(layer), q_full.view(T, -1))
        K.gemm(q, lw.w_uk_t, out=q_full.view(T, -1), x_group_koff=qhd, out_group_coff=lora + rope, k=nope)
        if fork:
            main.wait_stream(self.prep_stream)
        if prof is not None:
            prof.mark(layer, "attn.core")
        # verification batches (a few rows per decoding sequence) must take the same split path as plain
        # decode steps: equal split boundaries give bit-equal merges, hence the same greedy tokens
        cluster = ws.attn_splits in (2, 4, 8)       # splits merge through distributed shared memory
        ranges = [(0, T)]
        if b.n_tc_tiles:
            # sequences with many query rows: 128-row tiles on the tensor cores; the rest (decode and
            # verification rows of a mixed batch, short tails) keep the row-tile kernel
            K.mla_prefill_tc(q_full, self.pool.layer(layer), b.block_table, b.tc_tiles, b.n_tc_tiles,
                             self.pool.page_size, lora, rope, cfg.softmax_scale, ws.o_lat[:T], sink=lw.attn_sink)
            ranges = b.rest_ranges
        for r0, r1 in ranges:
            n = r1 - r0
            use_split = ws.attn_splits > 1 and n <= 4 * ws.decode_rows
            K.mla_attention(q_full[r0:r1], self.pool.layer(layer), b.block_table, b.row_seq[r0:r1], b.row_pos[r0:r1],
                            self.pool.page_size, lora, rope, cfg.softmax_scale, ws.o_lat[r0:r1],
                            splits=ws.attn_splits if use_split else 1,
                            split_tokens=self.split_tokens if use_split else (1 << 30) // 64 * 64,
                            ws=ws.attn_ws if (use_split and not cluster) else None, sink=lw.attn_sink,
                            decode_only=b.decode_only)
        if prof is not None:
            prof.mark(layer, "attn.uv")
        K.gemm(ws.o_lat[:T].view(T, -1), lw.w_uv, out=ws.attn_out[:T], x_group_koff=lora, out_group_coff=vd)
        return ws.attn_out[:T], lw.w_o

    def _fold_wanted(self) -> bool:
        if self.fold_decode == "auto":
            return self.tp is not None and self.tp.world >= 16
        return self.fold_decode == "1"

    def _build_fold(self, lw: LayerWeights):
        """(query weight, output weight) with the absorbed up-projections multiplied in, or None (quantised weights).
        Query side, per head: rows [W_UK^T @ W_q_nope ; W_q_rope] give the latent-space query and the rotary part
        in the layout the attention kernel reads.  Output side: W_o[:, head block] @ W_UV per head takes the latent
        attention output straight to the hidden size."""
        fold = None
        cfg = self.cfg
        wq = lw.w_q_b if cfg.q_lora_rank else lw.w_qkv_a
        plain = all(isinstance(t, torch.Tensor) for t in (wq, lw.w_o, lw.w_uk_t, lw.w_uv))
        if plain:
            hl, qhd, nope = self.w.heads_local, cfg.q_head_dim, cfg.qk_nope_dim
            lora, vd = cfg.kv_lora_rank, cfg.v_head_dim
            with torch.no_grad():
                qh = wq[:hl * qhd].view(hl, qhd, -1).float()
                q_abs = torch.bmm(lw.w_uk_t.float(), qh[:, :nope])                     # [hl, lora, in]
                wq_f = torch.cat([q_abs, qh[:, nope:]], dim=1).reshape(hl * (lora + qhd - nope), -1)
                if not cfg.q_lora_rank:
                    wq_f = torch.cat([wq_f, wq[hl * qhd:].float()], dim=0)            # the latent-kv rows follow
                wo = lw.w_o.float().view(lw.w_o.shape[0], hl, vd)
                wo_f = torch.einsum("ohv,hvl->ohl", wo, lw.w_uv.float()).reshape(lw.w_o.shape[0], hl * lora)
                fold = (wq_f.to(torch.bfloat16).contiguous(), wo_f.to(torch.bfloat16).contiguous())
        return fold

    def _attention_folded(self, lw: LayerWeights, fold, layer: int, xn: torch.Tensor, b: DeviceBatch, T: int):
        K, cfg, ws = self.K, self.cfg, self.ws
        hl, lora, rope = self.w.heads_local, cfg.kv_lora_rank, cfg.qk_rope_dim
        D = lora + rope
        wq_f, wo_f = fold
        if cfg.q_lora_rank:
            qkv = ws.qkv[:T]
            self._gemm(xn, lw.w_qkv_a, qkv, slot="xn")
            qa, ckv = qkv[:, :cfg.q_lora_rank], qkv[:, cfg.q_lora_rank:]
            self._norm(qa, lw.q_norm, T, ws.qn[:T], "a", None)
            q_rows = ws.q_full[:T].view(T, -1)
            K.gemm(ws.qn[:T], wq_f, out=q_rows)
        else:
            wide = ws.q_fold[:T]
            K.gemm(xn, wq_f, out=wide)
            q_rows, ckv = wide[:, :hl * D], wide[:, hl * D:]
        # the rotary part is rotated where it lies (each thread reads its pair before it writes it)
        K.mla_prep(q_rows, D, ckv, hl, lora, rope, lw.kv_norm, cfg.rms_eps, self.cos, self.sin,
                   b.positions, b.write_slot, self.pool.layer(layer), q_rows)
        q_full = q_rows.unflatten(1, (hl, D))
        cluster = ws.attn_splits in (2, 4, 8)
        use_split = ws.attn_splits > 1
        K.mla_attention(q_full, self.pool.layer(layer), b.block_table, b.row_seq[:T], b.row_pos[:T],
                        self.pool.page_size, lora, rope, cfg.softmax_scale, ws.o_lat[:T],
                        splits=ws.attn_splits if use_split else 1,
                        split_tokens=self.split_tokens if use_split else (1 << 30) // 64 * 64,
                        ws=ws.attn_ws if (use_split and not cluster) else None, sink=lw.attn_sink,
                        decode_only=b.decode_only)
        return ws.o_lat[:T].view(T, -1), wo_f

    def _moe_ntok(self, T: int) -> int:
        cfg = self.cfg
        est = T * cfg.topk / max(cfg.n_routed_experts, 1)
        return _pow2_at_least(2 * est, 16, 128)

    def _static_rows(self, lw: LayerWeights, T: int, layer: int) -> int:
        """Row-slot size of the static plan for this batch, 0 when the planned path must run (large batches,
        quantised or streamed experts, a hidden size the fused router does not take)."""
        ws = self.ws
        if not self.static_moe or layer < 0 or layer >= ws.route_cnt.shape[0] or self.cfg.hidden % 256:
            return 0
        if self.arena is not None and layer in self.arena.layers:
            return 0
        if isinstance(lw.e_w13, QuantWeight) and not lw.e_w13.native_mx:
            # plain 128 x 128 block-scaled FP8 experts take the static slots through the slot mode of the FP8 GEMM
            if lw.e_w13.group32 or not self.fp8_static or cfg_inter_bad(self.cfg):
                return 0
        for nt in ws.static_rows:
            if T <= nt:
                return nt
        return 0

    def _moe_local(self, lw: LayerWeights, xn: torch.Tensor, b: DeviceBatch, T: int, layer: int = -1, norm=None):
        """Router + local routed experts + shared experts -> ws.route_out filled for this rank.
        `norm` = (residual rows, sublayer output or None, new residual rows or None): `xn` has not been computed
        yet, the router kernel forms it (residual add + RMSNorm) in its prologue; static plan only."""
        K, cfg, ws = self.K, self.cfg, self.ws
        k, H = cfg.topk, cfg.hidden
        idx, wts = ws.topk_idx[:T], ws.topk_w[:T]
        ntok = self._moe_ntok(T)
        if isinstance(lw.e_w13, QuantWeight):
            ntok = min(ntok, 32)            # row-tile limit of the FP8 SwiGLU / group-scaled kernels
        plan = ws.plans[ntok]
        side = None
        static = self._static_rows(lw, T, layer)
        if norm is not None:
            assert static, "the fused norm + router kernel serves the static plan only"
            x_res, delta, res_out = norm
            K.router_append(x_res, lw.router_w, k, cfg.score_fn, ws.static_plans[static][layer], self.w.e_lo,
                            self.w.e_hi, idx, wts, ws.xg, bias=lw.router_bias, n_groups=cfg.n_groups,
                            topk_groups=cfg.topk_groups, normalize=cfg.norm_topk_prob, route_scale=cfg.route_scale,
                            hash_table=lw.hash_table, token_ids=b.token_ids, dst_slots=ws.slots,
                            norm_w=lw.ffn_norm, eps=cfg.rms_eps, delta=delta, res_out=res_out, norm_out=xn)
        # FP8 shared experts read the quantised normed rows: quantise before the fork
        kind13 = self._qkind(lw.w13)
        xq_n = self._quant_mx(xn, "xn_mx") if kind13 == "mx" else (self._quant(xn, "xn") if isinstance(lw.w13, QuantWeight)
                                                                      else None)
        if lw.w13 is not None:
            # The shared experts only need the normalised activations: fork them onto a second stream
            # (a parallel branch when captured in a graph) so they fill the SMs that the latency-bound
            # routing / planning kernels leave idle, and join before the reduction.
            side = self.side_stream
            main = torch.cuda.current_stream()
            side.wait_stream(main)
            with torch.cuda.stream(side):
                inter = lw.w13.shape[1] // 2
                if self.w.shared_replicated and self.tp is not None:
                    # the shared experts are held whole on every rank (for the token-dispatch form); in this
                    # replicated-activation form each rank multiplies its slice of their inner dimension
                    il = inter // self.tp.world
                    i0 = self.tp.rank * il
                    mid = ws.ffn_mid[:T, :il]
                    K.gemm(xn, lw.w13[:, i0:], out=mid, epilogue=K.EPI_SWIGLU, n_out=il, dual_offset=inter,
                           act_limit=cfg.swiglu_limit)
                    K.gemm(mid, lw.w2[:, :, i0:i0 + il], out=ws.route_out[:T][:, k])
                else:
                    mid = ws.ffn_mid[:T, :inter]
                    self._gemm(xn, lw.w13, mid, xq=xq_n, epilogue=K.EPI_SWIGLU, act_limit=cfg.swiglu_limit,
                               q_slot="mid" if self._qkind(lw.w2) == kind13 and kind13 else None)
                    self._gemm(mid, lw.w2, ws.route_out[:T][:, k], slot="mid")
                nl = self._prefetch_next
                if nl is not None and T <= ws.decode_rows:
                    # the next layer's attention weights (a few tens of MB, four latency-bound GEMMs) are pulled
                    # into L2 while the routed experts stream past them with the evict-first policy
                    for wt in (nl.w_qkv_a, nl.w_uk_t, nl.w_uv, nl.w_o):
                        if isinstance(wt, torch.Tensor):
                            K.l2_prefetch(wt, wt.numel() * wt.element_size())
        if static and isinstance(lw.e_w13, QuantWeight) and lw.e_w13.native_mx:
            # natively held MXFP4 experts: the normalised rows are quantised to MXFP8 once, the router gathers the
            # codes and scale bytes, the gate|up epilogue re-quantises the SwiGLU product for the down projection
            plan = ws.static_plans[static][layer]
            xq = self._quant_mx(xn, "xn_mx")
            (xgq, xgs), (hq, hs) = ws.act_q["xg_mx"], ws.act_q["hmid_mx"]
            K.router_append(xn, lw.router_w, k, cfg.score_fn, plan, self.w.e_lo, self.w.e_hi, idx, wts, None,
                            bias=lw.router_bias, n_groups=cfg.n_groups, topk_groups=cfg.topk_groups,
                            normalize=cfg.norm_topk_prob, route_scale=cfg.route_scale, hash_table=lw.hash_table,
                            token_ids=b.token_ids, dst_slots=ws.slots, quant_rows=(xq[0], xq[1], xgq, xgs))
            R, I = plan.cap_rows, cfg.moe_inter
            fp8w = lw.e_w13.packed is None          # e4m3 codes with replicated block scales instead of packed e2m1
            c13, c2 = (lw.e_w13.q, lw.e_w2.q) if fp8w else (lw.e_w13.packed, lw.e_w2.packed)
            # a slot is as high as the batch (every token may pick the same expert) but holds a few rows on
            # average: walk it in short tiles, so that stages, tensor work and epilogue follow the rows present
            sub = self.mx_slot_ntok
            kw = dict(slots=(plan.counts, static), ntok=sub) if (sub and static > sub and static % sub == 0) else {}
            self.Q.gemm_mxfp4(xgq[:R], xgs[:R], c13, lw.e_w13.sf, epilogue=K.EPI_SWIGLU, plan=plan,
                              act_limit=cfg.swiglu_limit, out_mx=(hq[:R, :I], hs[:R, :I // 32]), w_fp8=fp8w, **kw)
            self.Q.gemm_mxfp4(hq[:R, :I], hs[:R, :I // 32], c2, lw.e_w2.sf,
                              out=ws.route_out[:T].view(T * ws.slots, H), epilogue=K.EPI_SCATTER, plan=plan,
                              scatter_rows=T * ws.slots, w_fp8=fp8w, **kw)
            if side is not None:
                torch.cuda.current_stream().wait_stream(side)
            return idx
        if static and isinstance(lw.e_w13, QuantWeight):
            # block-scaled FP8 experts in the static slots: the router gathers the tokens' FP8 codes and scale bytes,
            # the FP8 GEMMs walk the slots (experts without rows are skipped), the gate|up epilogue re-quantises
            plan = ws.static_plans[static][layer]
            xq = xq_n if (xq_n is not None and kind13 == "fp8") else self._quant(xn, "xn")
            (xgq, xgs), (hq, hs) = ws.act_q["xg"], ws.act_q["hmid"]
            K.router_append(xn, lw.router_w, k, cfg.score_fn, plan, self.w.e_lo, self.w.e_hi, idx, wts, None,
                            bias=lw.router_bias, n_groups=cfg.n_groups, topk_groups=cfg.topk_groups,
                            normalize=cfg.norm_topk_prob, route_scale=cfg.route_scale, hash_table=lw.hash_table,
                            token_ids=b.token_ids, dst_slots=ws.slots, quant_rows=(xq[0], xq[1], xgq, xgs[:, :H // 128]))
            R, I = plan.cap_rows, cfg.moe_inter
            slots = (plan.counts, static)
            # 16-row tiles inside the slots: the epilogue of the block-scaled kernel rescales every k-block of
            # every row, so its cost follows the tile height, and most experts hold a few rows only
            self.Q.gemm_fp8(xgq[:R, :H], xgs[:R, :H // 128], lw.e_w13.q, lw.e_w13.scale, epilogue=K.EPI_SWIGLU,
                            slots=slots, act_limit=cfg.swiglu_limit, out_q=(hq[:R, :I], hs[:R, :I // 128]), ntok=16)
            self.Q.gemm_fp8(hq[:R, :I], hs[:R, :I // 128], lw.e_w2.q, lw.e_w2.scale,
                            out=ws.route_out[:T].view(T * ws.slots, H), epilogue=K.EPI_SCATTER, plan=plan,
                            slots=slots, scatter_rows=T * ws.slots, ntok=16)
            if side is not None:
                torch.cuda.current_stream().wait_stream(side)
            return idx
        if static:
            # no plan phase and no gather kernel: the router reserves rows in fixed per-expert slots
            plan = ws.static_plans[static][layer]
            if norm is None:
                K.router_append(xn, lw.router_w, k, cfg.score_fn, plan, self.w.e_lo, self.w.e_hi, idx, wts, ws.xg,
                                bias=lw.router_bias, n_groups=cfg.n_groups, topk_groups=cfg.topk_groups,
                                normalize=cfg.norm_topk_prob, route_scale=cfg.route_scale, hash_table=lw.hash_table,
                                token_ids=b.token_ids, dst_slots=ws.slots)
            R = plan.cap_rows
            K.gemm(ws.xg[:R], lw.e_w13, out=ws.hmid[:R], epilogue=K.EPI_SWIGLU, plan=plan, act_limit=cfg.swiglu_limit)
            K.gemm(ws.hmid[:R], lw.e_w2, out=ws.route_out[:T].view(T * ws.slots, H), epilogue=K.EPI_SCATTER,
                   plan=plan, scatter_rows=T * ws.slots)
            if side is not None:
                torch.cuda.current_stream().wait_stream(side)
            return idx
        if T <= self.fused_router_rows and H % 256 == 0:
            K.router_plan_fused(xn, lw.router_w, k, cfg.score_fn, plan, self.w.e_lo, self.w.e_hi, idx, wts,
                                ws.router_ctr, bias=lw.router_bias, n_groups=cfg.n_groups,
                                topk_groups=cfg.topk_groups, normalize=cfg.norm_topk_prob,
                                route_scale=cfg.route_scale, hash_table=lw.hash_table, token_ids=b.token_ids,
                                dst_slots=ws.slots)
        else:
            # one or two weight tiles: narrow row tiles so that the rows spread over the whole GPU
            K.gemm(xn, lw.router_w, out=ws.router_logits[:T],
                   ntok=32 if (T >= 1024 and lw.router_w.shape[0] <= 256) else None)
            K.router_topk(ws.router_logits[:T], k, cfg.score_fn, bias=lw.router_bias, n_groups=cfg.n_groups,
                          topk_groups=cfg.topk_groups, normalize=cfg.norm_topk_prob, route_scale=cfg.route_scale,
                          hash_table=lw.hash_table, token_ids=b.token_ids, out_idx=idx, out_w=wts)
            K.moe_plan(idx, wts, plan, self.w.e_lo, self.w.e_hi, dst_slots=ws.slots)
        streamed = self.arena is not None and layer in self.arena.layers
        K.gather_rows(xn, plan, ws.xg, cap_rows=T * k)
        if streamed:
            return self._moe_streamed(lw, plan, layer, T, side, idx)
        self._gemm(ws.xg[:T * k], lw.e_w13, ws.hmid[:T * k], slot="xg", epilogue=K.EPI_SWIGLU, plan=plan,
                   act_limit=cfg.swiglu_limit)
        route_out = ws.route_out[:T]
        plan2 = plan
        if (not isinstance(lw.e_w2, QuantWeight) and ntok == 128
                and T * k >= 160 * (self.w.e_hi - self.w.e_lo)):
            # prefill-sized expert loads: the scatter GEMM keeps one accumulator and takes 256-row tiles
            plan2 = ws.plans256 = K.moe_retile(plan, 256, getattr(ws, "plans256", None))
        # route r = t*k + s is written to row t*slots + s (the plan kernel emits that row index)
        self._gemm(ws.hmid[:T * k], lw.e_w2, route_out.view(T * ws.slots, H), slot="hmid", epilogue=K.EPI_SCATTER,
                   plan=plan2, scatter_rows=T * ws.slots)
        if side is not None:
            torch.cuda.current_stream().wait_stream(side)
        return idx

    def _moe_streamed(self, lw: LayerWeights, plan, layer: int, T: int, side, idx):
        """Routed experts of a layer whose weights live in an arena smaller than the expert set.  The batch's
        experts must be resident before the grouped GEMMs index the arena: read the per-expert row counts (one
        small device->host copy), then run the GEMM pair in waves of at most `frames` experts; in every wave the
        plan's tiles are translated from experts to slots, tiles of experts outside the wave get zero rows."""
        K, cfg, ws, arena = self.K, self.cfg, self.ws, self.arena
        k, H = cfg.topk, cfg.hidden
        counts = plan.counts[:self.w.e_hi - self.w.e_lo].cpu()
        need = counts.nonzero().flatten().tolist()
        if self.telemetry is not None:
            self.telemetry.record_counts(layer, counts.tolist(), T)
        if self.predictor is not None and not (self.wave_state or {}).get(layer, {}).get("done"):
            self.predictor.observe(layer, need)
        if self.async_stream:
            return self._moe_async(lw, plan, layer, T, side, idx, need)
        frames = arena.frames(layer)
        tg0, tr0 = plan.tile_group.clone(), plan.tile_rows.clone()
        route_out = ws.route_out[:T]
        for w0 in range(0, max(len(need), 1), frames):
            wave = need[w0:w0 + frames]
            if not wave:
                break
            if w0:
                plan.tile_group.copy_(tg0)
                plan.tile_rows.copy_(tr0)
            arena.ensure(layer, wave)
            arena.resolve_plan(layer, plan)
            # `_gemm` takes bf16 frames and quantised ones alike (the frames hold the experts' own form)
            self._gemm(ws.xg[:T * k], lw.e_w13, ws.hmid[:T * k], slot="xg", epilogue=K.EPI_SWIGLU, plan=plan,
                       act_limit=cfg.swiglu_limit)
            self._gemm(ws.hmid[:T * k], lw.e_w2, route_out.view(T * ws.slots, H), slot="hmid", epilogue=K.EPI_SCATTER,
                       plan=plan, scatter_rows=T * ws.slots)
            arena.release(layer)
        if side is not None:
            torch.cuda.current_stream().wait_stream(side)
        return idx

    def _moe_async(self, lw: LayerWeights, plan, layer: int, T: int, side, idx, need):
        """Streamed experts without blocking the engine.  The batch's experts are taken in waves of at most
        `frames` experts: a wave whose experts are all resident runs its GEMM pair on the leased frames and gives
        the leases back; a wave with a missing expert stops the layer here (`NeedExperts`) - its resident experts
        stay leased for the transaction, the experts of finished waves are remembered in `wave_state` together
        with their output rows, so the re-run of the layer after the resume restores those rows and goes on with
        the waves that are left.  With no more experts than frames this is a single wave whose leases are held
        until the transaction ends (`lease_sink`)."""
        from .expert_async import NeedExperts
        K, cfg, ws, arena = self.K, self.cfg, self.ws, self.arena
        k, H = cfg.topk, cfg.hidden
        frames = arena.frames(layer)
        single = len(need) <= frames
        state = self.wave_state.setdefault(layer, {"done": set(), "rows": None}) if self.wave_state is not None \
            else {"done": set(), "rows": None}
        route_out = ws.route_out[:T]
        if state["rows"] is not None:
            route_out[:, :k].copy_(state["rows"])            # output rows of the waves that ran before the park
            state["rows"] = None
        held = self.lease_sink.setdefault(layer, {}) if self.lease_sink is not None else {}
        pending = [e for e in need if e not in state["done"]]
        tg0 = tr0 = None
        if not single:
            tg0, tr0 = plan.tile_group.clone(), plan.tile_rows.clone()
        first = True
        while pending or first:
            wave = pending[:frames]
            held.update(arena.lease_resident(layer, [e for e in wave if e not in held]))
            missing = arena.missing(layer, wave)
            if missing:
                if state["done"]:
                    state["rows"] = route_out[:, :k].clone()
                if side is not None:
                    torch.cuda.current_stream().wait_stream(side)
                raise NeedExperts(layer, missing)
            if not first and tg0 is not None:
                plan.tile_group.copy_(tg0)
                plan.tile_rows.copy_(tr0)
            arena.resolve_plan(layer, plan)                  # experts that are not resident get zero-row tiles
            self._gemm(ws.xg[:T * k], lw.e_w13, ws.hmid[:T * k], slot="xg", epilogue=K.EPI_SWIGLU, plan=plan,
                       act_limit=cfg.swiglu_limit)
            self._gemm(ws.hmid[:T * k], lw.e_w2, route_out.view(T * ws.slots, H), slot="hmid",
                       epilogue=K.EPI_SCATTER, plan=plan, scatter_rows=T * ws.slots)
            first = False
            pending = pending[len(wave):]
            if not single:
                # the wave is done: its frames may go to the next wave's experts
                state["done"].update(wave)
                arena.release_leases(layer, [held.pop(e) for e in wave if e in held])
        if single and self.lease_sink is None:
            arena.release_leases(layer, list(held.values()))
        state["done"].clear()
        if side is not None:
            torch.cuda.current_stream().wait_stream(side)
        return idx

    def attach_ep(self, ep) -> None:
        """Use token-dispatch expert parallelism for the MoE layers of batches of world .. world * ep.tcap rows.
        Needs bf16 experts, shared experts replicated on every rank (`random_weights(replicate_shared=True)`)."""
        assert self.tp is not None and self.w.shared_replicated and ep.has_gather and ep.world == self.tp.world
        self.ep = ep
        R = ep.tcap
        cfg = self.cfg
        bf = dict(dtype=torch.bfloat16, device=self.device)
        self.ep_ws = {"xn": torch.zeros(R, cfg.hidden, **bf), "extra": torch.zeros(R, cfg.hidden, **bf),
                      "mid": torch.zeros(R, max(cfg.n_shared_experts * cfg.moe_inter, 8), **bf),
                      "logits": torch.zeros(R, cfg.n_routed_experts, dtype=torch.float32, device=self.device),
                      "idx": torch.zeros(R, cfg.topk, dtype=torch.int32, device=self.device),
                      "wts": torch.zeros(R, cfg.topk, dtype=torch.float32, device=self.device),
                      "out": torch.zeros(R, cfg.hidden, **bf)}

    def _ep_rows(self, T: int):
        """This rank's slice [lo, hi) of a batch of T rows (balanced, contiguous)."""
        W, r = self.ep.world, self.ep.rank
        base, rem = divmod(T, W)
        lo = r * base + min(r, rem)
        return lo, lo + base + (1 if r < rem else 0)

    def _use_ep(self, lw: LayerWeights, T: int) -> bool:
        return (self.ep is not None and lw.is_moe and self.ep.world <= T <= self.ep.world * self.ep.tcap
                and not isinstance(lw.e_w13, QuantWeight) and lw.hash_table is None)

    def _moe_dispatch(self, lw: LayerWeights, h_mid: torch.Tensor, b: DeviceBatch, T: int) -> torch.Tensor:
        """MoE layer under token-dispatch expert parallelism -> the batch's new residual rows [T, hidden] (a view
        of the gather buffer every rank's combine kernel pushed its slice into)."""
        K, cfg, ep, ws = self.K, self.cfg, self.ep, self.ep_ws
        lo, hi = self._ep_rows(T)
        n = hi - lo
        hs = h_mid[lo:hi]
        xn = ws["xn"][:n]
        K.add_rmsnorm(hs, lw.ffn_norm, cfg.rms_eps, norm_out=xn)
        extra = None
        side = None
        if lw.w13 is not None:
            side, main = self.side_stream, torch.cuda.current_stream()
            side.wait_stream(main)
            with torch.cuda.stream(side):
                inter = lw.w13.shape[1] // 2
                mid = ws["mid"][:n, :inter]
                K.gemm(xn, lw.w13, out=mid, epilogue=K.EPI_SWIGLU, act_limit=cfg.swiglu_limit)
                extra = ws["extra"][:n]
                K.gemm(mid, lw.w2, out=extra)
        logits = ws["logits"][:n]
        K.gemm(xn, lw.router_w, out=logits)
        idx, wts = ws["idx"][:n], ws["wts"][:n]
        K.router_topk(logits, cfg.topk, cfg.score_fn, bias=lw.router_bias, n_groups=cfg.n_groups,
                      topk_groups=cfg.topk_groups, normalize=cfg.norm_topk_prob, route_scale=cfg.route_scale,
                      out_idx=idx, out_w=wts)
        if side is not None:
            torch.cuda.current_stream().wait_stream(side)
        _, gathered = ep.forward(xn, idx, wts, lw.e_w13, lw.e_w2, residual=hs, extra=extra, out=ws["out"][:n],
                                 act_limit=cfg.swiglu_limit, allgather=True, gather_row0=lo)
        return gathered.view(-1, cfg.hidden)[:T]

    def _sp_active(self, T: int) -> bool:
        tp = self.tp
        if not self.sequence_parallel or tp is None or tp.world < 2 or T <= tp.fused_max_rows or self.ep is not None:
            return False
        if self.arena is not None:
            return False
        plain = lambda t: t is None or isinstance(t, torch.Tensor)
        return all(plain(getattr(lw, n)) for lw in self.w.layers
                   for n in ("w_qkv_a", "w_q_b", "w_o", "w13", "w2", "e_w13", "e_w2"))

    def layer_sp(self, lw: LayerWeights, layer: int, h_in: torch.Tensor, h_out: torch.Tensor, b: DeviceBatch,
                 T: int) -> torch.Tensor:
        """One layer on a row-sharded residual stream: only rows [lo, hi) of `h_in` / `h_out` / the result are this
        rank's and valid.  norm(rows) -> all-gather -> sublayer on all rows with this rank's heads / experts ->
        fp32 partial -> reduce-scatter + residual add on the rows.  Returns the buffer that holds the result."""
        K, cfg, ws, tp = self.K, self.cfg, self.ws, self.tp
        lo, hi = tp.row_range(T)
        n = hi - lo
        xn, xs = ws.xn[:T], ws.delta[:n]                    # delta: free in this form, holds the normalised slice
        self._norm(h_in[lo:hi], lw.attn_norm, n, xs, None, None)
        tp.all_gather(xs, xn, T)
        a, w_o = self._attention(lw, layer, xn, b, T)
        tp.gemm_reduce_scatter(a, w_o, h_in[lo:hi], h_out[lo:hi], T)
        self._norm(h_out[lo:hi], lw.ffn_norm, n, xs, None, None)
        tp.all_gather(xs, xn, T)
        if lw.is_moe:
            idx = self._moe_local(lw, xn, b, T, layer)
            tp.moe_reduce_scatter(ws.route_out[:T].view(T * ws.slots, cfg.hidden), ws.slots, cfg.topk, idx,
                                  self.w.e_lo, self.w.e_hi, h_out[lo:hi], h_in[lo:hi], T)
            return h_in
        inter = lw.w13.shape[1] // 2
        mid = ws.ffn_mid[:T, :inter]
        K.gemm(xn, lw.w13, out=mid, epilogue=K.EPI_SWIGLU, act_limit=cfg.swiglu_limit)
        tp.gemm_reduce_scatter(mid, lw.w2, h_out[lo:hi], h_in[lo:hi], T)
        return h_in

    def layer(self, lw: LayerWeights, layer: int, h_in: torch.Tensor, h_out: torch.Tensor, b: DeviceBatch,
              T: int, first_norm_done: bool = False, next_norm: Optional[torch.Tensor] = None) -> torch.Tensor:
        """h_in -> h_out (both bf16 [T, H]); returns h_out."""
        K, cfg, ws, tp = self.K, self.cfg, self.ws, self.tp
        xn = ws.xn[:T]
        if self.l2_prefetch_bytes and lw.is_moe and isinstance(lw.e_w13, torch.Tensor) and T <= ws.decode_rows:
            # Decode: the attention half of the layer is latency-bound and leaves HBM idle, and nearly every routed
            # expert will be read a few tens of microseconds from now.  Pull the head of the expert weights into
            # L2 meanwhile (side stream: a parallel branch of the graph), so the grouped GEMM starts on L2 hits.
            side, main = self.side_stream, torch.cuda.current_stream()
            side.wait_stream(main)
            with torch.cuda.stream(side):
                K.l2_prefetch(lw.e_w13, min(self.l2_prefetch_bytes, lw.e_w13.numel() * 2))
            if lw.w13 is None:                      # no shared-expert branch will join the side stream later
                main.wait_stream(side)
        # `first_norm_done`: the previous layer's last kernel already wrote this layer's normalised input to xn;
        # `next_norm` (single GPU): this layer's last kernel does the same for the next one
        prof = self.prof
        if prof is not None:
            prof.mark(layer, "attn.norm")
        if not first_norm_done:
            self._norm(h_in, lw.attn_norm, T, xn, "xn", self._qkind(lw.w_qkv_a))
        a, w_o = self._attention(lw, layer, xn, b, T)
        if prof is not None:
            prof.mark(layer, "attn.o_proj+norm")
        # what reads the post-attention norm: the dense FFN, or the shared experts and the static FP8 expert path
        ffn_q = self._qkind(lw.w13) or (self._qkind(lw.e_w13) if lw.is_moe else None)
        # decode-sized MoE layers: the post-attention residual add + RMSNorm runs in the router kernel's prologue
        route_norm = None
        use_ep = self._use_ep(lw, T)
        fuse_route = (not use_ep and self.fuse_router_norm and lw.is_moe and self._static_rows(lw, T, layer) > 0
                      and not isinstance(lw.w13, QuantWeight) and not isinstance(lw.e_w13, QuantWeight))
        if tp is None:
            self._gemm(a, w_o, ws.delta[:T], slot="a")
            if fuse_route:
                route_norm = (h_in, ws.delta[:T], h_out)
            else:
                self._norm(h_in, lw.ffn_norm, T, xn, "xn", ffn_q, delta=ws.delta[:T], res_out=h_out)
            h_mid = h_out
        else:
            if isinstance(w_o, QuantWeight):
                self._gemm(a, w_o, ws.delta[:T], slot="a")
                tp.add_allreduce(ws.delta[:T], residual=h_in, out=h_out, T=T)
            else:
                tp.gemm_allreduce(a, w_o, residual=h_in, out=h_out, T=T)
            if fuse_route:
                route_norm = (h_out, None, None)
            elif not use_ep:
                self._norm(h_out, lw.ffn_norm, T, xn, "xn", ffn_q)
            h_mid = h_out
        if prof is not None:
            prof.mark(layer, "moe" if lw.is_moe else "ffn")
        if self.tap is not None and self.tap.wants(layer, "attn_out"):
            self.tap.write(layer, "attn_out", h_mid)
        if use_ep:
            # the layer's result is the gathered tensor itself (symmetric memory the peers' combine kernels wrote)
            out = self._moe_dispatch(lw, h_mid, b, T)
            if prof is not None:
                prof.mark(layer, None)
            return out
        if lw.is_moe:
            idx = self._moe_local(lw, xn, b, T, layer, norm=route_norm)
            if self.route_observer is not None:
                self.route_observer(layer, idx, T)
            if prof is not None:
                prof.mark(layer, "moe.reduce")
            # slot `topk` holds the shared-expert row (zeros when the model has none)
            if tp is None and next_norm is not None:
                self._quantised.pop("xn", None)
                self._quantised.pop("xn_mx", None)
                K.moe_reduce_norm(ws.route_out[:T].view(T * ws.slots, cfg.hidden), ws.slots, cfg.topk, idx,
                                  self.w.e_lo, self.w.e_hi, T, cfg.hidden, h_mid, h_in, next_norm, xn, cfg.rms_eps)
            elif tp is None:
                K.moe_reduce(ws.route_out[:T].view(T * ws.slots, cfg.hidden), ws.slots, cfg.topk, idx,
                             self.w.e_lo, self.w.e_hi, T, cfg.hidden, residual=h_mid, out=h_in)
            else:
                tp.moe_reduce_allreduce(ws.route_out[:T].view(T * ws.slots, cfg.hidden), ws.slots, cfg.topk,
                                        idx, self.w.e_lo, self.w.e_hi, residual=h_mid, out=h_in, T=T)
            return h_in            # the layer's result lands back in the input buffer
        inter = lw.w13.shape[1] // 2
        mid = ws.ffn_mid[:T, :inter]
        self._gemm(xn, lw.w13, mid, slot="xn", epilogue=K.EPI_SWIGLU, act_limit=cfg.swiglu_limit,
                   q_slot="mid" if (self._qkind(lw.w2) and self._qkind(lw.w2) == self._qkind(lw.w13)) else None)
        if tp is None:
            self._gemm(mid, lw.w2, ws.delta[:T], slot="mid")
            # residual add is folded into the next consumer through a plain add+norm without a norm output
            if next_norm is not None:
                self._norm(h_mid, next_norm, T, xn, "xn", self._qkind(lw.w_qkv_a), delta=ws.delta[:T], res_out=h_in)
            else:
                K.add_rmsnorm(h_mid, None, cfg.rms_eps, delta=ws.delta[:T], res_out=h_in, want_norm=False)
        elif isinstance(lw.w2, QuantWeight):
            self._gemm(mid, lw.w2, ws.delta[:T], slot="mid")
            tp.add_allreduce(ws.delta[:T], residual=h_mid, out=h_in, T=T)
        else:
            tp.gemm_allreduce(mid, lw.w2, residual=h_mid, out=h_in, T=T)
        return h_in

    # -- whole model ---------------------------------------------------------------------
    def embed_rows(self, b: DeviceBatch, T: int) -> torch.Tensor:
        h = self.ws.h[0][:T]
        self.K.embedding(b.token_ids[:T], self.w.embed, out=h)
        return h

    def run_layers(self, h: torch.Tensor, b: DeviceBatch, T: int, start_layer: int = 0) -> torch.Tensor:
        """The layers this weight image holds (all of them, or one pipeline stage's share).  `h` is
        `ws.h[0][:T]` or is copied there."""
        ws = self.ws
        if h.data_ptr() != ws.h[0].data_ptr():
            self.M.copy_rows(ws.h[0], 0, h.contiguous())
        if ws.has_moe and ws.static_rows and T <= ws.static_rows[-1]:
            self.M.fill_(ws.route_cnt, 0)
        h, other = ws.h[0][:T], ws.h[1][:T]
        layers = self.w.layers
        if start_layer == 0 and self._sp_active(T):
            # every rank enters with the replicated rows, keeps its slice through the layers, and the slices are
            # gathered once at the end (the head reads arbitrary rows)
            for i, lw in enumerate(layers):
                h = self.layer_sp(lw, i, h, other, b, T)
            lo, hi = self.tp.row_range(T)
            self.tp.all_gather(h[lo:hi].clone(), h, T)
            return h
        fused = False                     # the previous layer wrote this layer's normalised input
        for i, lw in enumerate(layers):
            if i < start_layer:
                continue
            nxt = layers[i + 1].attn_norm if (self.fuse_next_norm and self.tp is None and i + 1 < len(layers)) else None
            self._prefetch_next = layers[i + 1] if (self.attn_prefetch and i + 1 < len(layers)) else None
            try:
                h = self.layer(lw, i, h, other, b, T, first_norm_done=fused, next_norm=nxt)
                fused = nxt is not None
            except Exception as exc:  # noqa: BLE001
                if hasattr(exc, "missing"):
                    exc.hidden = h.clone()      # the layer's input rows are intact: its last kernel writes them
                raise
            if self.tap is not None and self.tap.wants(i, "layer_out"):
                self.tap.write(i, "layer_out", h)
        if self.prof is not None:
            self.prof.mark(len(layers), None)       # ends the last layer's open stage
        return h

    def hidden_states(self, b: DeviceBatch, T: int, start_layer: int = 0, h0=None) -> torch.Tensor:
        """`start_layer` / `h0`: continue a forward that stopped at that layer with these input rows."""
        h = self.embed_rows(b, T) if h0 is None else h0
        return self.run_layers(h, b, T, start_layer)

    def head(self, h: torch.Tensor, b: DeviceBatch, final_norm: torch.Tensor, want_logits: bool = False,
             lm_head: Optional[torch.Tensor] = None):
        """Final norm + LM head + greedy token on the requested rows -> (next_id, next_val[, logits])."""
        K, cfg, ws, tp = self.K, self.cfg, self.ws, self.tp
        L = b.n_logit
        hl = ws.h_last[:L]
        self.M.gather_rows(h, b.logit_rows[:L], hl)
        K.add_rmsnorm(hl, final_norm, cfg.rms_eps, norm_out=ws.hn_last[:L])
        logits = ws.logits[:L]
        K.gemm(ws.hn_last[:L], self.w.lm_head if lm_head is None else lm_head, out=logits)
        K.argmax_chunked(logits, ws.argmax_scratch, ws.next_id[:L], ws.next_val[:L])
        if tp is not None:
            tp.argmax_across_vocab(ws.next_id[:L], ws.next_val[:L], self.w.vocab_lo, L)
        return ws.next_id[:L], ws.next_val[:L], (logits if want_logits else None)

    def forward(self, b: DeviceBatch, want_logits: bool = False, start_layer: int = 0, h0=None):
        """Runs the batch; returns (next_id [n_logit] int32, next_val, logits or None)."""
        T = b.token_ids.shape[0]
        assert T <= self.ws.max_rows and b.n_logit <= self.ws.max_logit_rows
        from ..ops import _lib
        start = _lib.LAUNCHES[0]
        h = self.hidden_states(b, T, start_layer, h0)
        self.last_hidden = h
        out = (None, None, None) if b.n_logit == 0 else self.head(h, b, self.w.final_norm, want_logits)
        self.launches = _lib.LAUNCHES[0] - start
        return out

    def mtp_forward(self, stage: int, h_prev: torch.Tensor, b: DeviceBatch):
        """MTP stage over rows carrying the next token ids; h_prev: main hidden states of those rows."""
        K, cfg, ws = self.K, self.cfg, self.ws
        m = self.w.mtp[stage]
        T = b.token_ids.shape[0]
        H = cfg.hidden
        x = ws.mtp_x[:T]
        if ws.has_moe and ws.static_rows and T <= ws.static_rows[-1]:
            self.M.fill_(ws.route_cnt[cfg.n_layers + stage], 0)
        # eh_proj input columns: [enorm(embedding) ; hnorm(previous hidden)], the order of published checkpoints
        K.add_rmsnorm(h_prev, m.hnorm, cfg.rms_eps, norm_out=x[:, H:])
        e = ws.h[1][:T]
        K.embedding(b.token_ids[:T], self.w.embed if m.embed is None else m.embed, out=e)
        K.add_rmsnorm(e, m.enorm, cfg.rms_eps, norm_out=x[:, :H])
        # h_prev (usually ws.h[0]) is consumed by now, so the projection may overwrite it
        h0 = ws.h[0][:T]
        self._gemm(x, m.eh_proj, h0, slot="a")
        h = self.layer(m.layer, cfg.n_layers + stage, h0, ws.h[1][:T], b, T)
        self.last_hidden = h
        return self.head(h, b, m.final_norm, lm_head=m.lm_head)


class DecodeGraph:
    """One captured decode step for a fixed row bucket.

    Inputs live in static device buffers (`self.batch`); `replay()` runs the whole step
    (embedding -> layers -> LM head -> greedy token) as one graph launch.  States mirror
    the reference's Cold -> Warm -> Captured graph cache
    (crates/ferrule-backend/src/cuda/graph.rs:70-150).
    """

    def __init__(self, fwd: CudaForward, rows: int, n_seqs: int, max_blocks: int,
                 batch: Optional[DeviceBatch] = None):
        dev = fwd.device
        i32 = dict(dtype=torch.int32, device=dev)
        self.fwd, self.rows = fwd, rows
        if batch is not None:
            batch.decode_only = True        # a decode graph carries one row per sequence
        self.batch = batch if batch is not None else DeviceBatch(torch.zeros(rows, **i32), torch.zeros(rows, **i32),
                                 torch.full((rows,), -1, dtype=torch.int64, device=dev),
                                 torch.zeros(rows, **i32), torch.full((rows,), -1, **i32),
                                 torch.zeros(n_seqs, max_blocks, **i32), torch.arange(rows, **i32), rows, rows, True)
        self.graph: Optional[torch.cuda.CUDAGraph] = None
        self.state = "cold"
        self.launches = 0

    def warm(self) -> None:
        self.fwd.forward(self.batch)
        self.launches = self.fwd.launches
        self.state = "warm"

    def capture(self) -> None:
        if self.state == "cold":
            s = torch.cuda.Stream()
            s.wait_stream(torch.cuda.current_stream())
            with torch.cuda.stream(s):
                self.warm()
            torch.cuda.current_stream().wait_stream(s)
        torch.cuda.synchronize()
        g = torch.cuda.CUDAGraph()
        with torch.cuda.graph(g):
            self.out = self.fwd.forward(self.batch)
        self.hidden = self.fwd.last_hidden          # static buffer the replay leaves the hidden states in
        self.graph, self.state = g, "captured"

    def replay(self):
        self.graph.replay()
        return self.out
