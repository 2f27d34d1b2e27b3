"""GLM-5.3-Flash on one B200 rank: device weight packing, state pools and the kernel chain.

The chain is the device twin of :class:`ferrite_b200.models.glm_ref.GlmReference` and of
the reference's per-layer device chains (``crates/ferrite-kernel/src/cuda.rs:3836-6298``,
``crates/ferrite-exec/src/tp.rs:2870-3393,5320-5500``), built from the hand-written
sm_100a kernels in ``csrc/kernels``.  Every buffer a kernel touches is allocated once, so a
forward pass can be captured in a CUDA graph and replayed; all per-step scalars (sequence
lengths, snapshot cursor, token ids) live in device memory and are advanced by graph nodes.
"""
from __future__ import annotations

import math
import zlib
from dataclasses import dataclass
from typing import Dict, List, Optional, Tuple

import torch

from .. import _lib
from ..config import EngineConfig, GlmConfig
from ..ops.reference import quant_fp8_block
from ..utils.switches import switches
from .glm_weights import init_kind, shard_weight, weight_layout

ROWMETA_BYTES = 32
HC_ACC = 25


# ---------------------------------------------------------------------------------------
# weight sources
# ---------------------------------------------------------------------------------------
class DictSource:
    """Weights from a name -> tensor dict (checkpoint or small random model)."""

    def __init__(self, weights: Dict[str, torch.Tensor], device):
        self.w, self.device = weights, device

    def get(self, name: str) -> torch.Tensor:
        return self.w[name].to(self.device)


class SyntheticSource:
    """Random-init weights generated on the device, tensor by tensor (no host copy).
    Matrices N(0, std); norm weights / HC scales 1; biases, A_log, dt_bias, HC bases 0."""

    def __init__(self, cfg: GlmConfig, device, seed: int = 0, std: float = 0.02, exact_shards: bool = False):
        self.layout = weight_layout(cfg)
        self.device, self.seed, self.std = device, seed, std
        # False: a rank draws its slice of the routed experts directly at the shard's width (fast; the model of a
        # TP=N run is then a different random model than that of a TP=1 run).  True: every rank draws the
        # full-width experts and slices them, so TP=N and TP=1 hold the same weights (token-identity checks).
        self.exact_shards = exact_shards

    def get(self, name: str) -> torch.Tensor:
        shape = self.layout[name]
        kind = init_kind(name)
        if kind == "zeros":
            return torch.zeros(shape, device=self.device)
        if kind == "ones":
            return torch.ones(shape, device=self.device)
        g = torch.Generator(device=self.device).manual_seed((self.seed << 32) ^ zlib.crc32(name.encode()))
        dt = torch.bfloat16 if len(shape) > 1 and shape[0] * shape[1] > (1 << 22) else torch.float32
        return torch.randn(shape, generator=g, device=self.device, dtype=dt) * self.std

    def expert_chunk(self, pfx: str, e0: int, e1: int, Il: int, H: int, rank: int = 0, world: int = 1):
        """Routed experts e0..e1 of one layer at the shard's width: (gate|up [n, 2*Il, H], down [n, H, Il]) in
        bf16; rank / world say which slice of the intermediate dim (only used with exact_shards)."""
        g = torch.Generator(device=self.device).manual_seed((self.seed << 32) ^ zlib.crc32(f"{pfx}.{e0}".encode()))
        n = e1 - e0
        if self.exact_shards and world > 1:
            I = Il * world
            full13 = torch.randn(n, 2 * I, H, generator=g, device=self.device, dtype=torch.bfloat16) * self.std
            full2 = torch.randn(n, H, I, generator=g, device=self.device, dtype=torch.bfloat16) * self.std
            lo, hi = rank * Il, (rank + 1) * Il
            a13 = torch.cat([full13[:, lo:hi], full13[:, I + lo:I + hi]], 1).contiguous()
            return a13, full2[:, :, lo:hi].contiguous()
        a13 = torch.randn(n, 2 * Il, H, generator=g, device=self.device, dtype=torch.bfloat16) * self.std
        a2 = torch.randn(n, H, Il, generator=g, device=self.device, dtype=torch.bfloat16) * self.std
        return a13, a2


@dataclass
class RowSet:
    """Static description of the rows of one forward pass: rows are grouped by sequence,
    groups are contiguous, row r of a group sits at position seq_len[slot] + off."""
    n: int
    n_groups: int
    row_slot: torch.Tensor
    row_off: torch.Tensor
    row_gsize: torch.Tensor
    group_first: torch.Tensor
    group_slot: torch.Tensor
    meta: torch.Tensor
    gsize_max: int


class GlmDeviceModel:
    def __init__(self, cfg: GlmConfig, ecfg: EngineConfig, src, rank: int = 0, world: int = 1,
                 device="cuda", allreduce=None, max_rows: int = 8, n_slots: int = 1,
                 num_pages: Optional[int] = None, layer_range: Optional[Tuple[int, int]] = None,
                 dcp_shard: Optional[Tuple[int, int]] = None):
        self.cfg, self.ecfg = cfg, ecfg
        # A pipeline stage of a layer-split (context-parallel) prefill group holds main layers [l0, l1) only
        # (crates/ferrite-kv/src/shard.rs:60-66 cp_layer_range); the MTP layer lives with the last stage.
        self.l0, self.l1 = layer_range if layer_range is not None else (0, cfg.num_layers)
        assert 0 <= self.l0 < self.l1 <= cfg.num_layers
        self.rank, self.world = rank, world
        self.dev = torch.device(device)
        self.K = _lib.lib()
        self.allreduce = allreduce  # callable(tensor_view[n,H]) summing across ranks, in place
        # GEMV + all-reduce + hyper-connection fold as one launch (None: separate kernels)
        self.fused = None
        from ..parallel.status import StatusArena
        self.arena = getattr(allreduce, "arena", None) or StatusArena(self.dev, 2048)
        mode = getattr(ecfg, "fuse_epilogue", "full")
        mode = {True: "full", False: "off"}.get(mode, mode)
        self.fuse_fold = mode == "full"
        if mode != "off" and (world > 1 or self.fuse_fold):
            if world > 1:
                self.fused = getattr(allreduce, "fused", None)
            else:
                from ..parallel.symm import FusedGemvAllReduce
                self.fused = FusedGemvAllReduce(self.dev, 0, 1, arena=self.arena, ar_group=switches().ar_group)
        self.dcp = None          # (d, n_dcp, DcpAttentionMerge): decode-context-parallel attention
        # (d, n): this rank of a decode-context-parallel group of n stores ONLY the latent pages p with p % n == d,
        # compactly (page p of a slot at latent page p // n): 1 / n of the latent cache per rank.  The indexer caches
        # stay whole on every rank (the top-k is global).
        self.dcp_shard = dcp_shard
        # decode GEMVs with at least this many output rows go to the tcgen05 split-K kernel (0 = never)
        sw = switches()
        self.tc_gemv_min_n, self.tc_gemv_max_n = sw.tc_gemv_min_n, sw.tc_gemv_max_n
        if sw.l2_ahead >= 0:
            self.K.lib.fb_set_l2_ahead(sw.l2_ahead)
        self.K.lib.fb_set_pdl(1 if sw.pdl else 0)
        self._tc_part = self._tc_ticket = None
        self._dense_tc, self._dense_act = {}, None     # per-row-count tile lists / f16 staging of the dense FFN's tcgen05 path
        self.fused_rows = 8      # forwards of up to this many rows use the fused epilogue; above 8 rows the kernel
                                 # would stream the weights once per 8-row window, where the tcgen05 GEMM streams them once
        self._fold_next = None   # (fn_next, front) while a hyper-connection site's sublayer runs; front = (scale,
                                 # base, ln_w) of the NEXT site when its hc_pre can ride in the closing GEMV
        self._folded = False
        self._pre_done = False   # the closing GEMV of the previous site already produced this site's x / post / comb
        self._wide_ready = False  # ... or left the partials (mix dots + Gram) for the column-parallel front kernel
        # sublayer-boundary fusion for decode rows (see csrc/kernels/gemv_ar.cu, gemv.cu, gdn.cu): next site's
        # hyper-connection front, SwiGLU as the down projection's activation source, routing as the router GEMV's
        # tail, the low-rank decay / gate projections inside the GatedDeltaNet kernel
        sw = switches()
        self.fuse_front = self.fuse_fold and cfg.hc_mult == 4 and sw.fuse_front
        self.fuse_route = mode != "off" and sw.fuse_route
        self.fuse_swiglu = mode != "off" and sw.fuse_swiglu
        self.gdn_own_fg = sw.gdn_own_fg
        self.hc_pre_wide = self.fuse_fold and cfg.hc_mult == 4 and sw.hc_pre_wide and not self.fuse_front
        self.route_ticket = self.arena.take(1, "route.ticket")
        self.max_rows = max_rows
        self.n_slots = n_slots
        self.num_pages_arg = num_pages
        la, ds = cfg.linear_attn, cfg.dsa
        assert la.num_heads % world == 0 and ds.num_heads % world == 0
        self.h_gdn = la.num_heads // world
        self.P = self.h_gdn * la.head_dim
        self.h_dsa = ds.num_heads // world
        self.kv_f32 = ecfg.kv_dtype == "f32"
        self.nbuf = (ecfg.mtp_n + 1) if ecfg.mtp_n > 1 else 1
        self.E_res = ecfg.experts_resident or cfg.n_routed_experts
        self.moe_by_expert = getattr(ecfg, "moe_shard", "inter") == "expert" and world > 1
        if self.moe_by_expert:
            assert cfg.n_routed_experts % world == 0 and not ecfg.experts_resident
            self.e_cnt = cfg.n_routed_experts // world
            self.e_lo = rank * self.e_cnt
        else:
            self.e_lo, self.e_cnt = 0, self.E_res
        self.tc_min_rows = 16  # row count from which dense bf16 projections use the tcgen05 GEMM
        self.tc_status = self.arena.status("tcgen05")       # bounded mbarrier waits of the tcgen05 kernels
        self.row_status = self.arena.status("rows")         # a sequence that reached the context limit (positions clamped)
        self.layers: List[dict] = []
        self.debug_hook = None  # callable(layer_index, site, ws, n) after each sublayer (eager runs only)
        self._pack(src)
        self._alloc_ws()
        self._alloc_state()

    # ------------------------------------------------------------------ packing
    def _sh(self, src, name):
        return shard_weight(name, src.get(name), self.rank, self.world)

    def _bf(self, t):
        return t.to(torch.bfloat16).contiguous()

    def _f(self, t):
        return t.float().contiguous()

    def _fp8(self, t):
        q, s = quant_fp8_block(t.float())
        return q.contiguous(), s.contiguous()

    def _pack_attn_linear(self, src, pfx, L):
        a = f"{pfx}.self_attn"
        cat = torch.cat([self._sh(src, f"{a}.qkv_proj.weight").float(), src.get(f"{a}.f_a_proj.weight").float(),
                         src.get(f"{a}.g_a_proj.weight").float(), self._sh(src, f"{a}.b_proj.weight").float()], 0)
        L["w_in"] = self._bf(cat)
        L["fg_b"] = self._bf(torch.cat([self._sh(src, f"{a}.f_b_proj.weight").float(),
                                        self._sh(src, f"{a}.g_b_proj.weight").float()], 0))
        L["conv_w"] = self._f(self._sh(src, f"{a}.qkv_conv1d.weight"))
        L["a_log"] = self._f(self._sh(src, f"{a}.A_log"))
        L["dt_bias"] = self._f(self._sh(src, f"{a}.dt_bias"))
        L["o_norm"] = self._f(src.get(f"{a}.o_norm.weight"))
        L["o_proj"] = self._bf(self._sh(src, f"{a}.o_proj.weight"))

    def _pack_attn_dsa(self, src, pfx, L):
        ds = self.cfg.dsa
        a = f"{pfx}.self_attn"
        cat = torch.cat([src.get(f"{a}.q_a_proj.weight").float(), src.get(f"{a}.kv_a_proj_with_mqa.weight").float(),
                         src.get(f"{a}.indexer.wk.weight").float(), src.get(f"{a}.indexer.weights_proj.weight").float(),
                         src.get(f"{a}.indexer.index_kpool_compress_gate").float()], 0)
        L["w_in"] = self._bf(cat)
        L["qa_ln"] = self._f(src.get(f"{a}.q_a_layernorm.weight"))
        L["kv_ln"] = self._f(src.get(f"{a}.kv_a_layernorm.weight"))
        L["kn_w"] = self._f(src.get(f"{a}.indexer.k_norm.weight"))
        L["kn_b"] = self._f(src.get(f"{a}.indexer.k_norm.bias"))
        L["ape"] = self._f(src.get(f"{a}.indexer.index_kpool_compress_ape"))
        L["w_q"] = self._bf(torch.cat([self._sh(src, f"{a}.q_b_proj.weight").float(),
                                       src.get(f"{a}.indexer.wq_b.weight").float()], 0))
        kvb = self._sh(src, f"{a}.kv_b_proj.weight").float()
        dk, dv, DL = ds.qk_nope_head_dim, ds.v_head_dim, ds.kv_lora_rank
        kvb = kvb.view(self.h_dsa, dk + dv, DL)
        # absorbed forms: q_abs[h] = Wk_h^T q_h (rows = latent dim), o_h = Wv_h ctx_h
        L["wk_abs"] = self._bf(kvb[:, :dk, :].transpose(1, 2).reshape(self.h_dsa * DL, dk))
        L["wv_abs"] = self._bf(kvb[:, dk:, :].reshape(self.h_dsa * dv, DL))
        L["o_proj"] = self._bf(self._sh(src, f"{a}.o_proj.weight"))

    def _pack_mlp_dense(self, src, pfx, L):
        g = self._sh(src, f"{pfx}.mlp.gate_proj.weight").float()
        u = self._sh(src, f"{pfx}.mlp.up_proj.weight").float()
        d = self._sh(src, f"{pfx}.mlp.down_proj.weight").float()
        if self.ecfg.fp8_experts:
            L["d13"], L["d13s"] = self._fp8(torch.cat([g, u], 0))
            L["d2"], L["d2s"] = self._fp8(d)
        else:
            L["d13"], L["d2"] = self._bf(torch.cat([g, u], 0)), self._bf(d)
        L["I_dense"] = g.shape[0]

    def _pack_mlp_moe(self, src, pfx, L):
        cfg = self.cfg
        E, Er = cfg.n_routed_experts, self.E_res
        bias = self._f(src.get(f"{pfx}.mlp.gate.e_score_correction_bias")).clone()
        if Er < E:
            bias[Er:] = -1e30  # experts that are not resident can never be routed to
        L["gate_bias"] = bias
        sg = self._sh(src, f"{pfx}.mlp.shared_expert.gate_proj.weight").float()
        su = self._sh(src, f"{pfx}.mlp.shared_expert.up_proj.weight").float()
        L["gate_s13"] = self._bf(torch.cat([src.get(f"{pfx}.mlp.gate.weight").float(), sg, su], 0))
        L["s2"] = self._bf(self._sh(src, f"{pfx}.mlp.shared_expert.down_proj.weight"))
        L["I_shared"] = sg.shape[0]
        by_e = self.moe_by_expert
        Il = cfg.moe_intermediate_size if by_e else cfg.moe_intermediate_size // self.world
        e_lo, Er = (self.e_lo, self.e_cnt) if by_e else (0, Er)   # the experts this rank stores (local index = id - e_lo)
        get = (lambda name: src.get(name)) if by_e else (lambda name: self._sh(src, name))
        H = cfg.hidden_size
        w13 = torch.empty(Er, 2 * Il, H, dtype=torch.float8_e4m3fn, device=self.dev)
        s13 = torch.empty(Er, (2 * Il + 127) // 128, (H + 127) // 128, device=self.dev)
        w2 = torch.empty(Er, H, Il, dtype=torch.float8_e4m3fn, device=self.dev)
        s2 = torch.empty(Er, (H + 127) // 128, (Il + 127) // 128, device=self.dev)
        chunk = getattr(src, "expert_chunk", None)
        if chunk is not None and (2 * Il) % 128 == 0 and H % 128 == 0:
            step = 16
            for e0 in range(0, Er, step):
                e1 = min(Er, e0 + step)
                a13, a2 = chunk(pfx, e_lo + e0, e_lo + e1, Il, H, *((0, 1) if by_e else (self.rank, self.world)))
                q, s = quant_fp8_block(a13.view(-1, H))
                w13[e0:e1], s13[e0:e1] = q.view(e1 - e0, 2 * Il, H), s.view(e1 - e0, -1, s.shape[1])
                q, s = quant_fp8_block(a2.view(-1, Il))
                w2[e0:e1], s2[e0:e1] = q.view(e1 - e0, H, Il), s.view(e1 - e0, -1, s.shape[1])
        else:
            for e in range(Er):
                g = get(f"{pfx}.mlp.experts.{e_lo + e}.gate_proj.weight").float()
                u = get(f"{pfx}.mlp.experts.{e_lo + e}.up_proj.weight").float()
                d = get(f"{pfx}.mlp.experts.{e_lo + e}.down_proj.weight").float()
                w13[e], s13[e] = quant_fp8_block(torch.cat([g, u], 0))
                w2[e], s2[e] = quant_fp8_block(d)
        L["w13"], L["s13s"], L["w2"], L["s2s"] = w13, s13, w2, s2
        L["I_moe"] = Il

    def _pack(self, src):
        cfg = self.cfg
        self.embed = self._bf(src.get("model.embed_tokens.weight"))
        # the head is sliced by vocab rows when the ranks can merge their argmax (cross-rank exchange);
        # every rank then streams 1/world of the largest matrix of the model
        head = src.get("lm_head.weight")
        self.xargmax = getattr(self.allreduce, "argmax", None) if self.world > 1 else None
        self.vocab_off = 0
        if self.xargmax is not None and head.shape[0] % (self.world * 16) == 0:
            vl = head.shape[0] // self.world
            self.vocab_off = self.rank * vl
            head = head[self.vocab_off:self.vocab_off + vl]
        else:
            self.xargmax = None
        self.lm_head = self._bf(head)
        self.final_norm = self._f(src.get("model.norm.weight"))
        n_total = cfg.num_layers + cfg.num_nextn_predict_layers
        for i in range(n_total):
            pfx = f"model.layers.{i}"
            owned = (self.l0 <= i < self.l1) if i < cfg.num_layers else self.l1 == cfg.num_layers
            if not owned:
                self.layers.append(None)      # another stage's layer: no weights here
                continue
            L = {"idx": i, "dsa": cfg.is_dsa(i), "moe": cfg.is_moe(i), "mtp": i >= cfg.num_layers}
            L["ln1"] = self._f(src.get(f"{pfx}.input_layernorm.weight"))
            L["ln2"] = self._f(src.get(f"{pfx}.post_attention_layernorm.weight"))
            if not L["mtp"] and cfg.mhc:
                for site in ("attn", "ffn"):
                    L[f"hc_{site}_fn"] = self._f(src.get(f"{pfx}.hc_{site}_fn"))
                    L[f"hc_{site}_scale"] = self._f(src.get(f"{pfx}.hc_{site}_scale"))
                    L[f"hc_{site}_base"] = self._f(src.get(f"{pfx}.hc_{site}_base"))
            if L["mtp"]:
                L["enorm"] = self._f(src.get(f"{pfx}.enorm.weight"))
                L["hnorm"] = self._f(src.get(f"{pfx}.hnorm.weight"))
                L["eh_proj"] = self._bf(src.get(f"{pfx}.eh_proj.weight"))
                L["head_norm"] = self._f(src.get(f"{pfx}.shared_head.norm.weight"))
            (self._pack_attn_dsa if L["dsa"] else self._pack_attn_linear)(src, pfx, L)
            (self._pack_mlp_moe if L["moe"] else self._pack_mlp_dense)(src, pfx, L)
            if L["dsa"]:
                L["family"] = cfg.dsa_family(i)
            else:
                L["gdn_index"] = cfg.linear_layers.index(i)
            self.layers.append(L)

    # ------------------------------------------------------------------ buffers
    def _z(self, *shape, dtype=torch.float32):
        return torch.zeros(*shape, dtype=dtype, device=self.dev)

    def _act(self, ld, split=True):
        return Act(self.dev, self.max_rows, ld, split)

    def _alloc_ws(self):
        cfg, la, ds, M = self.cfg, self.cfg.linear_attn, self.cfg.dsa, self.max_rows
        H = cfg.hidden_size
        ws = {}
        ws["R0"] = self._z(M, cfg.hc_mult, H)
        ws["R1"] = self._z(M, cfg.hc_mult, H)
        ws["R"] = ws["R0"]
        ws["x"] = self._act(H)         # sublayer input (normed), f32 + split planes
        ws["y"] = self._z(M, H)        # sublayer output
        ws["res"] = self._z(M, H)      # plain residual (MTP layer)
        ws["post"] = self._z(M, cfg.hc_mult)
        ws["comb"] = self._z(M, cfg.hc_mult * cfg.hc_mult)
        ws["hc_acc"] = self._z(M, HC_ACC)
        self.ld_gdn = 3 * self.P + 2 * la.low_rank + self.h_gdn
        self.ld_gdn += (-self.ld_gdn) % 8
        ws["gdn_proj"] = self._act(self.ld_gdn)
        ws["gdn_fg"] = self._z(M, 2 * self.P)
        ws["gdn_core"] = self._act(self.P)
        self.ld_dsa = ds.q_lora_rank + ds.kv_lora_rank + 2 * ds.index_head_dim + ds.index_n_heads
        ws["dsa_proj"] = self._z(M, self.ld_dsa + (-self.ld_dsa) % 4)
        ws["dsa_qa"] = self._act(ds.q_lora_rank)
        ws["dsa_wi"] = self._z(M, ds.index_n_heads)
        self.ld_qq = self.h_dsa * ds.qk_nope_head_dim + ds.index_n_heads * ds.index_head_dim
        ws["dsa_qq"] = self._act(self.ld_qq)
        ws["dsa_qabs"] = self._z(M, self.h_dsa * ds.kv_lora_rank)
        self.max_pools = (self.ecfg.max_ctx + ds.index_kpool - 1) // ds.index_kpool + 1
        ws["dsa_scores"] = self._z(M, self.max_pools)
        ws["dsa_idx"] = self._z(M, ds.idx_width + ds.index_kpool, dtype=torch.int32)
        ws["dsa_cnt"] = self._z(M, dtype=torch.int32)
        self.nsplit = 32 if self.h_dsa * ds.kv_lora_rank >= 4096 else 2
        ws["dsa_opart"] = self._z(M, self.nsplit, self.h_dsa, ds.kv_lora_rank)
        ws["dsa_ml"] = self._z(M, self.nsplit, self.h_dsa, 2)
        ws["dsa_ctx"] = self._act(self.h_dsa * ds.kv_lora_rank)
        ws["dsa_ov"] = self._act(self.h_dsa * ds.v_head_dim)
        owned = [L for L in self.layers if L is not None]
        Imax = max([L.get("I_dense", 0) for L in owned] + [L.get("I_shared", 0) for L in owned] + [8])
        Imax += (-Imax) % 8
        ws["gu"] = self._z(M, 2 * Imax)
        ws["act"] = self._act(Imax)
        Ismax = max([L.get("I_shared", 0) for L in owned] + [1])
        ws["moe_lg"] = self._z(M, cfg.n_routed_experts + 2 * Ismax)
        ws["moe_ids"] = self._z(M, cfg.num_experts_per_tok, dtype=torch.int32)
        ws["moe_wts"] = self._z(M, cfg.num_experts_per_tok)
        Il = max([L.get("I_moe", 0) for L in owned] + [8])
        Il += (-Il) % 8
        ws["moe_act"] = self._z(M, cfg.num_experts_per_tok, Il)
        ws["moe_act_s"] = torch.zeros(4, M * cfg.num_experts_per_tok, Il, dtype=torch.int16, device=self.dev)
        self.gdn_chunk_rows = switches().gdn_chunk_rows   # groups of at least this many rows take the WY-chunked scan
        self.moe_group_rows = 8      # more rows than this: group (row, slot) pairs by expert
        # from this row count the grouped experts run as tcgen05 GEMMs (fp8 weights widened to bf16 in shared memory,
        # csrc/kernels/fp8w_gemm.cu); below it the mma.sync grouped kernels (0 = never)
        self.moe_tc_rows = switches().moe_tc_rows
        if M >= self.moe_tc_rows > 0:
            npair = M * cfg.num_experts_per_tok
            i32 = lambda *s_: torch.zeros(*s_, dtype=torch.int32, device=self.dev)
            ws["tc_pos"], ws["tc_wts"] = i32(npair), self._z(npair)
            ws["tc_counts"], ws["tc_offsets"] = i32(512), i32(513)
            ws["tc_tiles"], ws["tc_ntiles"] = i32(512 + npair // 32 + 1, 4), i32(1)
            ws["tc_x"] = torch.zeros(npair, H, dtype=torch.float16, device=self.dev)
            ws["tc_h"] = self._z(npair, 2 * Il)
            ws["tc_act"] = torch.zeros(npair, Il, dtype=torch.float16, device=self.dev)
        if M > self.moe_group_rows:
            npair = M * cfg.num_experts_per_tok
            ws["moe_gpairs"] = torch.zeros(npair * 8, dtype=torch.int32, device=self.dev)
            ws["moe_gexp"] = torch.zeros(npair, dtype=torch.int32, device=self.dev)
            ws["moe_ngrp"] = torch.zeros(1, dtype=torch.int32, device=self.dev)
            ws["moe_ypair"] = torch.zeros(npair, cfg.hidden_size, device=self.dev)
        ws["h_final"] = self._z(M, H)
        ws["xh"] = self._act(H)
        ws["logits"] = self._z(M, self.lm_head.shape[0])
        ws["amax_part"] = self._z(M * 64, dtype=torch.int64)
        ws["mtp_in"] = self._act(2 * H)
        ws["mtp_hout"] = self._z(M, H)
        self.ws = ws

    def _alloc_state(self):
        cfg, la, ds = self.cfg, self.cfg.linear_attn, self.cfg.dsa
        S, nb = self.n_slots, self.nbuf
        ng = len(cfg.linear_layers)
        self.gdn_state = self._z(ng, S, nb, self.h_gdn, la.head_dim, la.head_dim)
        self.conv_state = self._z(ng, S, nb, 3 * self.P, la.conv_kernel - 1)
        ps = ds.page_size
        self.max_pages = (self.ecfg.max_ctx + ps - 1) // ps
        # default: static identity paging (slot s owns its own range); with an explicit page
        # count the table is filled by the caller's page allocator (page 0 = scratch page)
        self.num_pages = self.num_pages_arg or S * self.max_pages
        nf = cfg.n_dsa_families
        kvdt = torch.float32 if self.kv_f32 else torch.bfloat16
        self.lat_table = None
        lat_pages = self.num_pages
        if self.dcp_shard is not None:
            d, nd = self.dcp_shard
            assert not self.num_pages_arg, "compact DCP storage is built on static identity paging"
            self.lat_pages_slot = (self.max_pages + nd - 1) // nd
            lat_pages = S * self.lat_pages_slot
            lp = torch.arange(self.max_pages)
            row = torch.where(lp % nd == d, lp // nd, torch.full_like(lp, -1))
            tab = torch.stack([torch.where(row >= 0, row + s_ * self.lat_pages_slot, row) for s_ in range(S)])
            self.lat_table = tab.to(torch.int32).to(self.dev).contiguous()
        self.lat_cache = torch.zeros(nf, lat_pages, ps, ds.kv_lora_rank, dtype=kvdt, device=self.dev)
        self.kidx_cache = self._z(nf, self.num_pages, ps, ds.index_head_dim)
        self.kgate_cache = self._z(nf, self.num_pages, ps, ds.index_head_dim)
        self.pool_cache = self._z(nf, self.num_pages, ps // ds.index_kpool, ds.index_head_dim)
        # static identity paging: slot s owns pages [s*max_pages, (s+1)*max_pages)
        if self.num_pages_arg:
            self.page_table = torch.zeros(S, self.max_pages, dtype=torch.int32, device=self.dev)
        else:
            self.page_table = torch.arange(self.num_pages, dtype=torch.int32, device=self.dev).view(S, self.max_pages).contiguous()
        self.main_len = self._z(S, dtype=torch.int32)
        self.mtp_len = self._z(S, dtype=torch.int32)
        self.cur = self._z(S, dtype=torch.int32)

    def reset_slot(self, slot: int):
        self.gdn_state[:, slot].zero_()
        self.conv_state[:, slot].zero_()
        self.main_len[slot] = 0
        self.mtp_len[slot] = 0
        self.cur[slot] = 0

    def make_rows(self, slots: List[int], gsizes: List[int]) -> RowSet:
        rs, ro, rg, gf = [], [], [], []
        for s, g in zip(slots, gsizes):
            gf.append(len(rs))
            for o in range(g):
                rs.append(s); ro.append(o); rg.append(g)
        n = len(rs)
        assert n <= self.max_rows, (n, self.max_rows)
        t = lambda v: torch.tensor(v, dtype=torch.int32, device=self.dev)
        return RowSet(n, len(slots), t(rs), t(ro), t(rg), t(gf), t(list(slots)),
                      torch.zeros(n * ROWMETA_BYTES, dtype=torch.uint8, device=self.dev), max(gsizes))

    # ------------------------------------------------------------------ op helpers
    def gemv(self, w, x, out, m, N, K, ldx=None, ldo=None, group_rows=0, accumulate=False, scales=None,
             xcol=0, ocol=0, omask=0):
        """out[:m, ocol:ocol+N] (+)= x[:m, xcol:...] . w^T.  x / out may be :class:`Act` buffers
        (f32 + split planes) or plain f32 tensors.  Rows go eight at a time; each chunk streams
        the weights once.  The tensor-core kernel runs when the input has split planes and K
        fits its k-block; otherwise the SIMT kernel reads the f32 copy."""
        xa = x if isinstance(x, Act) else None
        oa = out if isinstance(out, Act) else None
        xf = xa.f if xa else x
        of = oa.f if oa else out
        ldx = ldx if ldx is not None else (xa.ld if xa else K)
        ldo = ldo if ldo is not None else (oa.ld if oa else N)
        fp8 = scales is not None
        kb = 128 if fp8 else 64
        use_mma = xa is not None and xa.s is not None and K % kb == 0 and group_rows % 16 == 0 and ldx % 8 == 0
        tc_min_n = getattr(self, "tc_gemv_min_n", 0)
        tc_max_n = getattr(self, "tc_gemv_max_n", 0)   # 9-16 rows: matrices with few row tiles leave the plain GEMM with few CTAs
        tc_gemv = (use_mma and not fp8 and group_rows == 0 and 8 < m <= 16 and K % 64 == 0
                   and ((tc_min_n and N >= tc_min_n) or (tc_max_n and N <= tc_max_n)))
        if (use_mma and not fp8 and group_rows > 0 and group_rows % 128 == 0 and N % group_rows == 0
                and m >= self.tc_min_rows):
            # a block-diagonal projection at prefill row counts: the tcgen05 GEMM picks each tile's x columns by group
            xp = _lib.ctypes.c_void_p(xa.s.data_ptr() + xcol * 2)
            op = _lib.ctypes.c_void_p(of.data_ptr() + ocol * 4)
            self.K.call("fb_gemm_tc_bf16_grouped", w, xp, ldx, op, ldo, m, N, K, group_rows, int(accumulate), self.tc_status)
            if oa is not None and omask:
                self.K.call("fb_split_rows", op, ldo, _lib.ctypes.c_void_p(oa.s.data_ptr() + ocol * 2), ldo, oa.plane,
                            omask, m, N)
            return
        if use_mma and not fp8 and group_rows == 0 and m >= self.tc_min_rows and not tc_gemv:
            # prefill-sized row counts: TMA + tcgen05 GEMM over the bf16 high plane of the activations
            xp = _lib.ctypes.c_void_p(xa.s.data_ptr() + xcol * 2)
            op = _lib.ctypes.c_void_p(of.data_ptr() + ocol * 4)
            self.K.call("fb_gemm_tc_bf16", w, xp, ldx, op, ldo, m, N, K, int(accumulate), self.tc_status)
            if oa is not None and omask:
                self.K.call("fb_split_rows", op, ldo, _lib.ctypes.c_void_p(oa.s.data_ptr() + ocol * 2), ldo, oa.plane,
                            omask, m, N)
            return
        if tc_gemv or (use_mma and not fp8 and group_rows == 0 and m <= 16 and tc_min_n and N >= tc_min_n and K % 64 == 0):
            # decode-sized rows of a large matrix: TMA + tcgen05 split-K GEMV (bf16 hi + lo activation planes)
            tiles = (N + 127) // 128
            nsplit = max(1, min(K // 256, -(-296 // tiles)))
            need = tiles * nsplit * 16 * 128
            if self._tc_part is None or self._tc_part.numel() < need or self._tc_ticket.numel() < tiles:
                self._tc_part = torch.zeros(max(need, 4 << 20), device=self.dev)
                self._tc_ticket = torch.zeros(max(tiles, 2048), dtype=torch.int32, device=self.dev)
            xp = _lib.ctypes.c_void_p(xa.s.data_ptr() + xcol * 2)
            op = _lib.ctypes.c_void_p(of.data_ptr() + ocol * 4)
            self.K.call("fb_gemv_tc_bf16", w, xp, ldx, xa.plane, op, ldo, m, N, K, int(accumulate), nsplit, self._tc_part,
                        self._tc_ticket, self.tc_status)
            if oa is not None and omask:
                self.K.call("fb_split_rows", op, ldo, _lib.ctypes.c_void_p(oa.s.data_ptr() + ocol * 2), ldo, oa.plane,
                            omask, m, N)
            return
        if use_mma:
            # one launch: the kernel's second grid dimension walks the 8-row windows
            op = _lib.ctypes.c_void_p(of.data_ptr() + ocol * 4)
            osb = ((_lib.ctypes.c_void_p(oa.s.data_ptr() + ocol * 2), ldo, oa.plane, omask) if oa is not None and omask
                   else (None, 0, 0, 0))
            xp = _lib.ctypes.c_void_p(xa.s.data_ptr() + xcol * 2)
            if fp8:
                self.K.call("fb_gemv_mma_fp8", w, scales, xp, ldx, xa.plane, op, ldo, m, N, K, accumulate, *osb)
            else:
                self.K.call("fb_gemv_mma_bf16", w, xp, ldx, xa.plane, op, ldo, m, N, K, group_rows, accumulate, *osb)
            return
        for r0 in range(0, m, 8):
            mm = min(8, m - r0)
            op = _lib.ctypes.c_void_p(of.data_ptr() + (r0 * ldo + ocol) * 4)
            if oa is not None and omask:
                osb = (_lib.ctypes.c_void_p(oa.s.data_ptr() + (r0 * ldo + ocol) * 2), ldo, oa.plane, omask)
            else:
                osb = (None, 0, 0, 0)
            if use_mma:
                xp = _lib.ctypes.c_void_p(xa.s.data_ptr() + (r0 * ldx + xcol) * 2)
                if fp8:
                    self.K.call("fb_gemv_mma_fp8", w, scales, xp, ldx, xa.plane, op, ldo, mm, N, K, accumulate, *osb)
                else:
                    self.K.call("fb_gemv_mma_bf16", w, xp, ldx, xa.plane, op, ldo, mm, N, K, group_rows, accumulate, *osb)
                continue
            xp = _lib.ctypes.c_void_p(xf.data_ptr() + (r0 * ldx + xcol) * 4)
            if fp8:
                self.K.call("fb_gemv_fp8", w, scales, xp, ldx, op, ldo, mm, N, K, group_rows, accumulate)
            else:
                self.K.call("fb_gemv_bf16", w, xp, ldx, op, ldo, mm, N, K, group_rows, accumulate)
            if osb[0] is not None:
                self.K.call("fb_split_rows", op, ldo, *osb, mm, N)

    def _argmax(self, out_ids, n, V):
        """Greedy ids of ws['logits'][:n] (this rank's vocab slice when the head is sliced)."""
        ws = self.ws
        if self.xargmax is None:
            self.K.call("fb_argmax", ws["logits"], V, ws["amax_part"], out_ids, None, n, V, 1, 0)
        else:
            self.xargmax(ws["logits"], V, ws["amax_part"], n, V, self.vocab_off, out_ids)

    def _reduce(self, y, n):
        if self.world > 1:
            step = max(1, getattr(self.allreduce, "max_elems", y[:n].numel()) // y.shape[1])
            for r0 in range(0, n, step):   # the one-shot all-reduce takes a bounded payload per launch
                self.allreduce(y[r0:min(n, r0 + step)])

    def _out_gemv(self, w, x, n, N, K, ldx=None, scales=None, accumulate=False, swiglu=None):
        """The GEMV that ends a sublayer: ws['y'] = x . w^T (+ ws['y']) summed over the ranks.  When
        the fused kernel applies, the all-reduce and (inside a hyper-connection site) hc_post, the
        next site's mix dots and its whole hc_pre ride in the same launch; otherwise GEMV and
        all-reduce run separately and the caller's _hc_post_mix / _hc_pre do the rest.
        swiglu = (gu, ld, up_off): x = SwiGLU of the f32 [gate | up] rows `gu`; the fused kernel applies it
        while it loads its activations, the fallback runs the SwiGLU kernel into `x` first."""
        ws, cfg = self.ws, self.cfg
        fold, self._fold_next = self._fold_next, None
        if not self.fuse_fold:
            fold = None
        xa = x if isinstance(x, Act) else None
        ldx = ldx if ldx is not None else (xa.ld if xa else K)
        kb = 128 if scales is not None else 64
        ok = (self.fused is not None and xa is not None and xa.s is not None and n <= self.fused_rows and K % kb == 0
              and ldx % 8 == 0 and N % 4 == 0 and (self.world == 1 or 8 * N <= self.fused.max_elems)
              and (self.world > 1 or fold is not None or (swiglu is not None and self.fuse_swiglu)))
        sw = None
        if swiglu is not None:
            gu, ldg, up_off = swiglu
            if ok and self.fuse_swiglu and ldg % 4 == 0 and up_off % 4 == 0 and gu.data_ptr() % 16 == 0:
                sw = (gu, ldg, up_off, float(cfg.swiglu_limit))
            else:
                self.K.call("fb_swiglu_split", gu, ldg, xa.f, *xa.sp(3, ld=K), n, K, float(cfg.swiglu_limit))
        if not ok:
            gar = getattr(self.allreduce, "gemm_fused", None) if self.world > 1 else None
            if (gar is not None and scales is None and xa is not None and xa.s is not None and n >= self.tc_min_rows
                    and K % 8 == 0 and ldx % 8 == 0 and ws["y"].shape[1] % 4 == 0 and gar.fits(n, N)):
                # prefill rows: TMA + tcgen05 GEMM with the two-shot all-reduce in its epilogue (one launch)
                gar(w, xa.s, ldx, ws["y"], ws["y"].shape[1], n, N, K, accumulate)
                return
            self.gemv(w, x, ws["y"], n, N, K, ldx=ldx, scales=scales, accumulate=accumulate)
            self._reduce(ws["y"], n)
            return
        f = front = None
        want_gram = False
        if fold is not None:
            rin = ws["R"]
            rout = ws["R1"] if rin is ws["R0"] else ws["R0"]
            f = (rin, rout, ws["post"], ws["comb"], fold[0], ws["hc_acc"], cfg.hc_mix)
            ws["R"] = rout
            self._folded = True
            nxt = fold[1] if len(fold) > 1 else None
            if nxt is not None and fold[0] is not None and self.fuse_front and n <= 8 and N == cfg.hidden_size:
                xo = ws["x"]
                front = (nxt[0], nxt[1], nxt[2], ws["post"], ws["comb"], xo.f, xo.sp(3), float(cfg.rms_norm_eps),
                         float(cfg.hc_eps), cfg.hc_sinkhorn_iters)
                self._pre_done = True
            elif fold[0] is not None and self.hc_pre_wide and n <= 8 and N == cfg.hidden_size and N // 16 <= 512:
                self._wide_ready = want_gram = True
        self.fused(w, scales, None if sw is not None else xa.s, ldx, xa.plane, ws["y"], N, n, N, K, accumulate,
                   fold is None or self.debug_hook is not None, f, swiglu=sw, front=front, gram=want_gram)

    # ------------------------------------------------------------------ sublayers
    def _attn_linear(self, L, rs: RowSet, snapshots: bool):
        cfg, la, ws, n = self.cfg, self.cfg.linear_attn, self.ws, rs.n
        H, P, r = cfg.hidden_size, self.P, la.low_rank
        proj = ws["gdn_proj"]
        own_fg = self.gdn_own_fg and rs.gsize_max <= 8 and r <= 128 and r % 16 == 0
        self.gemv(L["w_in"], ws["x"], proj, n, L["w_in"].shape[0], H, omask=0 if own_fg else 1)
        if not own_fg:
            self.gemv(L["fg_b"], proj, ws["gdn_fg"], n, 2 * P, r, group_rows=P, xcol=3 * P)
        gi = L["gdn_index"]
        core = ws["gdn_core"]
        if not snapshots and rs.gsize_max >= self.gdn_chunk_rows > 0 and la.head_dim in (64, 128):
            # prefill-sized groups: WY-chunked scan (32 tokens per step of matrix products instead of 32 serial steps)
            self.K.call("fb_gdn_chunk", proj.f, self.ld_gdn, ws["gdn_fg"], View(ws["gdn_fg"], P), 2 * P, L["conv_w"],
                        L["a_log"], L["dt_bias"], L["o_norm"], self.gdn_state[gi], self.conv_state[gi], self.cur, rs.meta,
                        rs.group_first, rs.n_groups, core.f, P, self.h_gdn, la.head_dim, 3 * P + 2 * r, self.nbuf,
                        float(la.gate_lower_bound), float(cfg.rms_norm_eps), *core.sp(1))
            self._out_gemv(L["o_proj"], core, n, H, P)
            return
        self.K.call("fb_gdn_fused", proj.f, self.ld_gdn, ws["gdn_fg"], View(ws["gdn_fg"], P), 2 * P, L["conv_w"],
                    L["a_log"], L["dt_bias"], L["o_norm"], self.gdn_state[gi], self.conv_state[gi], self.cur, rs.meta,
                    rs.group_first, rs.n_groups, core.f, P, self.h_gdn, la.head_dim, 3 * P + 2 * r,
                    self.nbuf, int(snapshots), float(la.gate_lower_bound), float(cfg.rms_norm_eps), *core.sp(1),
                    L["fg_b"] if own_fg else None, 3 * P, r, rs.gsize_max)
        self._out_gemv(L["o_proj"], core, n, H, P)

    def _attn_dsa(self, L, rs: RowSet):
        cfg, ds, ws, n = self.cfg, self.cfg.dsa, self.ws, rs.n
        H = cfg.hidden_size
        f = L["family"]
        QL, DL, ID, IH = ds.q_lora_rank, ds.kv_lora_rank, ds.index_head_dim, ds.index_n_heads
        dk, dv, hl = ds.qk_nope_head_dim, ds.v_head_dim, self.h_dsa
        ldp = ws["dsa_proj"].shape[1]
        self.gemv(L["w_in"], ws["x"], ws["dsa_proj"], n, self.ld_dsa, H, ldo=ldp)
        pt, mp, ps = self.page_table, self.max_pages, ds.page_size
        qa, qq, ctx, ov = ws["dsa_qa"], ws["dsa_qq"], ws["dsa_ctx"], ws["dsa_ov"]
        self.K.call("fb_dsa_prep", ws["dsa_proj"], ldp, L["qa_ln"], L["kv_ln"], L["kn_w"], L["kn_b"], qa.f,
                    ws["dsa_wi"], self.lat_cache[f], self.kidx_cache[f], self.kgate_cache[f], rs.meta, pt, self.lat_table,
                    mp, ps, n, QL, DL, ID, IH, float(cfg.rms_norm_eps), int(self.kv_f32), *qa.sp(1))
        lt = self.lat_table if self.lat_table is not None else pt     # the latent cache's own page table
        self.K.call("fb_dsa_pool", self.kidx_cache[f], self.kgate_cache[f], L["ape"], self.pool_cache[f], rs.meta,
                    pt, mp, ps, n, ID, ds.index_kpool)
        self.gemv(L["w_q"], qa, qq, n, self.ld_qq, QL, omask=1)
        self.K.call("fb_dsa_scores", View(qq.f, hl * dk), self.ld_qq, ws["dsa_wi"], self.pool_cache[f],
                    ws["dsa_scores"], self.max_pools, rs.meta, pt, mp, ps, n, IH, ID, ds.index_kpool, self.max_pools)
        ldi = ws["dsa_idx"].shape[1]
        self.K.call("fb_dsa_select", ws["dsa_scores"], self.max_pools, ws["dsa_idx"], ldi, ws["dsa_cnt"], rs.meta,
                    n, ds.index_kpool, ds.select_pools)
        self.gemv(L["wk_abs"], qq, ws["dsa_qabs"], n, hl * DL, dk, group_rows=DL)
        d_, n_ = (self.dcp[0], self.dcp[1]) if self.dcp is not None else (0, 1)
        # key splits: decode rows need them to fill the GPU; a prefill chunk has a CTA per row already, and every
        # split re-reads the row's 64 x 512 query and adds a partial to merge (1024 rows x 32 splits: 3.3 ms + 0.7 ms
        # per layer against a fraction of that unsplit)
        ns = self.nsplit if n <= 64 else (2 if n < 256 else 1)
        if DL == 512 and not self.kv_f32:   # tensor-core form (bf16 latents)
            self.K.call("fb_dsa_attn_partial_tc", ws["dsa_qabs"], self.lat_cache[f], ws["dsa_idx"], ldi, ws["dsa_cnt"],
                        ws["dsa_opart"], ws["dsa_ml"], rs.meta, lt, mp, ps, n, hl, DL, ns, d_, n_,
                        float(dk ** -0.5))
        else:
            self.K.call("fb_dsa_attn_partial", ws["dsa_qabs"], self.lat_cache[f], ws["dsa_idx"], ldi, ws["dsa_cnt"],
                        ws["dsa_opart"], ws["dsa_ml"], rs.meta, lt, mp, ps, n, hl, DL, ns, d_, n_,
                        float(dk ** -0.5), int(self.kv_f32))
        if self.dcp is None:
            self.K.call("fb_dsa_attn_merge", ws["dsa_opart"], ws["dsa_ml"], ctx.f, None, n, hl, DL, ns, 1,
                        *ctx.sp(1))
        else:
            # decode context parallel: this rank attends over its own pages (page % n_dcp == d) of the
            # global top-k list; the merge kernel exchanges the partials with the peers and finishes
            merge = self.dcp[2]
            merge(ws["dsa_opart"], ws["dsa_ml"], ctx.f, n, hl, DL, ns, ctx.sp(1))
        self.gemv(L["wv_abs"], ctx, ov, n, hl * dv, DL, group_rows=dv, omask=1)
        self._out_gemv(L["o_proj"], ov, n, H, hl * dv)

    def _ffn_dense(self, L, n):
        cfg, ws = self.cfg, self.ws
        H, I = cfg.hidden_size, L["I_dense"]
        ldg = ws["gu"].shape[1]
        act = ws["act"]
        if (L.get("d13s") is not None and 0 < self.moe_tc_rows <= n and H % 128 == 0 and I % 128 == 0 and "tc_x" in ws
                and ws["y"].shape[1] % 4 == 0):
            # prefill rows: the e4m3 dense FFN as a one-expert case of the grouped W8A16 tcgen05 GEMM
            K = self.K
            self._fold_next = None
            t = self._dense_tc.get(n)
            if t is None:
                bn = 32 if n <= 32 else 64 if n <= 64 else 128
                mt = (n + bn - 1) // bn + 1
                i32 = lambda *a: torch.zeros(*a, dtype=torch.int32, device=self.dev)
                t = {"tiles": i32(mt, 4), "nt": i32(1), "off": i32(2), "bn": bn, "mt": mt,
                     "cnt": torch.tensor([n], dtype=torch.int32, device=self.dev),
                     "iota": torch.arange(n, dtype=torch.int32, device=self.dev), "ones": torch.ones(n, device=self.dev)}
                K.call("fb_mx_tiles", t["cnt"], 1, bn, t["tiles"], t["nt"], t["off"], mt)
                self._dense_tc[n] = t
            if self._dense_act is None or self._dense_act.shape[1] < max(I, H):
                self._dense_act = torch.zeros(self.max_rows, max(I, H), dtype=torch.float16, device=self.dev)
            xh = self._dense_act
            K.call("fb_scatter_rows_f16", ws["x"].f, ws["x"].ld, t["iota"], 1, n, H, xh)
            K.call("fb_fp8w_gemm_grouped", L["d13"], L["d13s"], xh, t["tiles"], t["nt"], t["mt"], ws["gu"], ldg, n, 1,
                   2 * I, H, t["bn"], self.tc_status)
            K.call("fb_swiglu_rows_f16", ws["gu"], ldg, t["ones"], t["cnt"], n, I, float(cfg.swiglu_limit), xh)
            K.call("fb_fp8w_gemm_grouped", L["d2"], L["d2s"], xh, t["tiles"], t["nt"], t["mt"], ws["y"], ws["y"].shape[1],
                   n, 1, H, I, t["bn"], self.tc_status)
            self._reduce(ws["y"], n)
            return
        self.gemv(L["d13"], ws["x"], ws["gu"], n, 2 * I, H, ldo=ldg, scales=L.get("d13s"))
        # SwiGLU rides in the down projection's activation load (or runs as its own kernel, rows packed with stride I)
        self._out_gemv(L["d2"], act, n, H, I, ldx=I, scales=L.get("d2s"), swiglu=(ws["gu"], ldg, I))

    def _ffn_moe(self, L, n):
        cfg, ws = self.cfg, self.ws
        H, E, topk = cfg.hidden_size, cfg.n_routed_experts, cfg.num_experts_per_tok
        Il, Is = L["I_moe"], L["I_shared"]
        ldl = ws["moe_lg"].shape[1]
        act, x = ws["act"], ws["x"]
        tail = (self.fuse_route and n <= 8 and E <= 384 and H % 64 == 0 and x.ld % 8 == 0 and x.s is not None
                and not self.tc_gemv_min_n)
        if tail:
            # router logits | shared gate | shared up in one GEMV whose last router CTA also routes the rows; the
            # shared expert's SwiGLU is applied by its down projection (below)
            self.K.call("fb_gemv_mma_bf16_route", L["gate_s13"], x.s, x.ld, x.plane, ws["moe_lg"], ldl, n, E + 2 * Is, H,
                        L["gate_bias"], ws["moe_ids"], ws["moe_wts"], self.route_ticket, E, topk,
                        float(cfg.routed_scaling_factor))
        else:
            self.gemv(L["gate_s13"], x, ws["moe_lg"], n, E + 2 * Is, H, ldo=ldl)  # router logits | shared gate|up
            # routing and the shared expert's SwiGLU read the same GEMV output row: one launch
            self.K.call("fb_moe_route_swiglu", ws["moe_lg"], ldl, L["gate_bias"], ws["moe_ids"], ws["moe_wts"], n, E, topk,
                        float(cfg.routed_scaling_factor), act.f, *act.sp(1, ld=Is), Is, float(cfg.swiglu_limit))
        # routed experts write y, the shared expert's down projection adds to it and carries the
        # all-reduce (and the hyper-connection fold) in its epilogue
        if H % 128 == 0 and Il % 128 == 0 and 0 < self.moe_tc_rows <= n and self.e_cnt <= 512:
            # prefill-sized row counts on tcgen05: pairs sorted by expert, f16 rows scattered to their sorted places,
            # gate | up GEMM, weighted SwiGLU, down GEMM, slot-ordered combine; every expert's weights stream once
            K = self.K
            npairs = n * topk
            bn = 32 if npairs <= 32 * self.e_cnt else 64 if npairs <= 64 * self.e_cnt else 128
            mt = ws["tc_tiles"].shape[0]
            K.call("fb_mx_sort", ws["moe_ids"], ws["moe_wts"], npairs, self.e_lo, self.e_cnt, bn, ws["tc_pos"], ws["tc_wts"],
                   ws["tc_counts"], ws["tc_offsets"], ws["tc_tiles"], ws["tc_ntiles"], mt)
            K.call("fb_scatter_rows_f16", x.f, x.ld, ws["tc_pos"], topk, n, H, ws["tc_x"])
            K.call("fb_fp8w_gemm_grouped", L["w13"], L["s13s"], ws["tc_x"], ws["tc_tiles"], ws["tc_ntiles"], mt, ws["tc_h"],
                   ws["tc_h"].shape[1], npairs, self.e_cnt, 2 * Il, H, bn, self.tc_status)
            K.call("fb_swiglu_rows_f16", ws["tc_h"], ws["tc_h"].shape[1], ws["tc_wts"], View(ws["tc_offsets"], self.e_cnt),
                   npairs, Il, float(cfg.swiglu_limit), ws["tc_act"])
            K.call("fb_fp8w_gemm_grouped", L["w2"], L["s2s"], ws["tc_act"], ws["tc_tiles"], ws["tc_ntiles"], mt, ws["moe_ypair"],
                   H, npairs, self.e_cnt, H, Il, bn, self.tc_status)
            K.call("fb_mx_combine", ws["moe_ypair"], H, ws["tc_pos"], topk, ws["y"], ws["y"].shape[1], n, H, 0)
        elif H % 128 == 0 and Il % 128 == 0 and n > self.moe_group_rows:
            # prefill-sized row counts: pairs grouped by expert, each expert's weights stream once per group
            mas = ws["moe_act_s"]
            ld_as, plane_as = mas.shape[2], mas.shape[1] * mas.shape[2]
            mg = n * topk
            self.K.call("fb_moe_group", ws["moe_ids"], n * topk, self.e_lo, self.e_cnt, ws["moe_gpairs"], ws["moe_gexp"],
                        ws["moe_ngrp"], mg)
            self.K.call("fb_moe_gate_up_grp", L["w13"], L["s13s"], x.s, x.ld, x.plane, ws["moe_wts"], ws["moe_gpairs"],
                        ws["moe_gexp"], ws["moe_ngrp"], mas, ld_as, plane_as, mg, topk, Il, H, float(cfg.swiglu_limit))
            self.K.call("fb_moe_down_grp", L["w2"], L["s2s"], mas, ld_as, plane_as, ws["moe_gpairs"], ws["moe_gexp"],
                        ws["moe_ngrp"], ws["moe_ypair"], mg, Il, H)
            self.K.call("fb_moe_sum_pairs", ws["moe_ypair"], ws["moe_ids"], ws["y"], H, n, topk, H, self.e_lo, self.e_cnt, 0)
        elif H % 128 == 0 and Il % 128 == 0:
            mas = ws["moe_act_s"]
            ld_as, plane_as = mas.shape[2], mas.shape[1] * mas.shape[2]
            self.K.call("fb_moe_gate_up_mma", L["w13"], L["s13s"], x.s, x.ld, x.plane, ws["moe_ids"], ws["moe_wts"],
                        mas, ld_as, plane_as, n, topk, Il, H, self.e_lo, self.e_cnt, float(cfg.swiglu_limit))
            self.K.call("fb_moe_down_mma", L["w2"], L["s2s"], mas, ld_as, plane_as, ws["moe_ids"], ws["y"], H, n,
                        topk, Il, H, self.e_lo, self.e_cnt, 0, None, 0, 0, 0)
        else:
            self.K.call("fb_moe_gate_up_fp8", L["w13"], L["s13s"], x.f, H, ws["moe_ids"], ws["moe_act"], n, topk,
                        Il, H, self.e_lo, self.e_cnt, float(cfg.swiglu_limit))
            self.K.call("fb_moe_down_fp8", L["w2"], L["s2s"], ws["moe_act"], ws["moe_ids"], ws["moe_wts"], ws["y"],
                        H, n, topk, Il, H, self.e_lo, self.e_cnt, 0)
        self._out_gemv(L["s2"], act, n, H, Is, ldx=Is, accumulate=True,
                       swiglu=(View(ws["moe_lg"], E), ldl, Is) if tail else None)

    def _attn(self, L, rs, snapshots):
        if L["dsa"]:
            self._attn_dsa(L, rs)
        else:
            self._attn_linear(L, rs, snapshots)

    def _ffn(self, L, n):
        if L["moe"]:
            self._ffn_moe(L, n)
        else:
            self._ffn_dense(L, n)

    def _hc_pre(self, L, site, ln, n, first=False):
        """Coefficients + contraction + RMSNorm of one site; its mix dots are already in hc_acc."""
        cfg, ws = self.cfg, self.ws
        if self._pre_done:   # the previous site's closing GEMV already left x, post and comb
            self._pre_done = False
            return
        x = ws["x"]
        if self._wide_ready:   # partials (mix dots, sum of squares, Gram) are waiting: column-parallel front
            self._wide_ready = False
            part, gram, part_n, ld = self.fused.wide_partials()
            self.K.call("fb_hc_pre_wide", ws["R"], part, gram, part_n, ld, L[f"hc_{site}_scale"], L[f"hc_{site}_base"], ln,
                        x.f, ws["post"], ws["comb"], n, cfg.hidden_size, cfg.hc_mix, float(cfg.rms_norm_eps),
                        float(cfg.hc_eps), cfg.hc_sinkhorn_iters, *x.sp(3))
            return
        # the first site of a forward has no producer: its mix dots are in hc_acc, never in the partial buffers
        self.K.call("fb_hc_pre_apply", ws["R"], ws["hc_acc"], L[f"hc_{site}_scale"], L[f"hc_{site}_base"], ln, None,
                    x.f, ws["post"], ws["comb"], n, cfg.hidden_size, cfg.hc_mult, float(cfg.rms_norm_eps),
                    float(cfg.hc_eps), cfg.hc_sinkhorn_iters, *x.sp(3),
                    *(self.fused.partials() if self.fused is not None and n <= self.fused_rows and not first
                      else (None, None, 0)))

    def _hc_post_mix(self, fn_next, n, first=False):
        """hc_post of the finished site fused with the mix dots of the next one; the residual
        stream ping-pongs between two buffers because the mix blocks re-read the old one."""
        cfg, ws = self.cfg, self.ws
        if self._folded:   # the sublayer's last GEMV already did hc_post and the mix dots
            self._folded = False
            return
        rin = ws["R"]
        rout = ws["R1"] if rin is ws["R0"] else ws["R0"]
        if first:
            self.K.call("fb_hc_post_mix", rin, rin, None, None, None, fn_next, ws["hc_acc"], n, cfg.hidden_size, cfg.hc_mix)
            return
        self.K.call("fb_hc_post_mix", rin, rout, ws["y"], ws["post"], ws["comb"], fn_next, ws["hc_acc"], n,
                    cfg.hidden_size, cfg.hc_mix)
        ws["R"] = rout

    # ------------------------------------------------------------------ passes
    def main_forward(self, rs: RowSet, ids: torch.Tensor, snapshots: bool = False, advance: bool = True,
                     judges: Optional[torch.Tensor] = None, head_from: int = 0):
        """Main model over the rows of ``rs`` (token ids on the device).  Leaves logits in
        ws['logits'][:n], the pre-norm contracted residual in ws['h_final'][:n] and, when
        ``judges`` is given, the greedy token of every row there."""
        cfg, ws, n, K = self.cfg, self.ws, rs.n, self.K
        H = cfg.hidden_size
        K.call("fb_prep_rows", rs.row_slot, rs.row_off, rs.row_gsize, self.main_len, rs.meta, n, self.ecfg.max_ctx,
               self.row_status)
        ws["R"] = ws["R0"]
        if self.l0 == 0:
            K.call("fb_embed_expand", ids, self.embed, ws["R"], n, H, cfg.hc_mult, cfg.vocab_size)
        # a later pipeline stage finds the residual streams of its rows in ws["R0"][:n] (the previous stage's output)
        main = self.layers[self.l0:self.l1]
        self._hc_post_mix(main[0]["hc_attn_fn"], n, first=True)
        for li, L in enumerate(main):
            self._hc_pre(L, "attn", L["ln1"], n, first=(li == 0))
            self._fold_next = (L["hc_ffn_fn"], (L["hc_ffn_scale"], L["hc_ffn_base"], L["ln2"]))
            self._attn(L, rs, snapshots)
            self._hc_post_mix(L["hc_ffn_fn"], n)
            if self.debug_hook:
                self.debug_hook(L["idx"], "attn", ws, n)
            self._hc_pre(L, "ffn", L["ln2"], n)
            nl = main[li + 1] if li + 1 < len(main) else None
            fn_next = nl["hc_attn_fn"] if nl is not None else None
            self._fold_next = (fn_next, (nl["hc_attn_scale"], nl["hc_attn_base"], nl["ln1"]) if nl is not None else None)
            self._ffn(L, n)
            self._hc_post_mix(fn_next, n)
            if self.debug_hook:
                self.debug_hook(L["idx"], "ffn", ws, n)
        if self.l1 == cfg.num_layers:
            xh = ws["xh"]
            K.call("fb_hc_head", ws["R"], self.final_norm, ws["h_final"], xh.f, n, H, cfg.hc_mult,
                   float(cfg.rms_norm_eps), *xh.sp(1))
            V = self.lm_head.shape[0]
            nh = n - head_from  # the head runs on rows [head_from, n); their logits land in rows [0, nh)
            if nh > 0:
                self.gemv(self.lm_head, xh, ws["logits"], nh, V, H, xcol=head_from * H)
                if judges is not None:
                    self._argmax(View(judges, head_from), nh, V)
        if advance:
            K.call("fb_advance_rows", rs.meta, None, self.main_len, n)

    def mtp_forward(self, rs: RowSet, ids: torch.Tensor, h_prev: torch.Tensor, out_ids: Optional[torch.Tensor],
                    head_from: int = 0, advance: bool = True):
        """The MTP layer over rows (token, h_prev).  ws['mtp_hout'][:n] = its residual output;
        out_ids[r - head_from] = greedy draft token of row r >= head_from."""
        cfg, ws, n, K = self.cfg, self.ws, rs.n, self.K
        H = cfg.hidden_size
        L = self.layers[cfg.num_layers]
        eps = float(cfg.rms_norm_eps)
        K.call("fb_prep_rows", rs.row_slot, rs.row_off, rs.row_gsize, self.mtp_len, rs.meta, n, self.ecfg.max_ctx,
               self.row_status)
        mi, x, xh = ws["mtp_in"], ws["x"], ws["xh"]
        K.call("fb_mtp_prep", ids, self.embed, h_prev, L["enorm"], L["hnorm"], mi.f, n, H, cfg.vocab_size, eps, *mi.sp(1))
        self.gemv(L["eh_proj"], mi, ws["res"], n, H, 2 * H)
        K.call("fb_rmsnorm", ws["res"], None, None, L["ln1"], x.f, n, H, H, H, eps, *x.sp(3))
        self._attn_dsa(L, rs)
        K.call("fb_rmsnorm", ws["res"], ws["y"], ws["res"], L["ln2"], x.f, n, H, H, H, eps, *x.sp(3))
        self._ffn_moe(L, n)
        K.call("fb_rmsnorm", ws["res"], ws["y"], ws["mtp_hout"], L["head_norm"], xh.f, n, H, H, H, eps, *xh.sp(1))
        nh = n - head_from
        if out_ids is not None and nh > 0:
            V = self.lm_head.shape[0]
            self.gemv(self.lm_head, xh, ws["logits"], nh, V, H, xcol=head_from * H)
            self._argmax(out_ids, nh, V)
        if advance:
            K.call("fb_advance_rows", rs.meta, None, self.mtp_len, n)


class Act:
    """An activation buffer [M, ld]: an f32 copy plus the four 16-bit split planes
    (bf16 hi/lo, f16 hi/lo) that the tensor-core GEMVs read."""

    def __init__(self, dev, M: int, ld: int, split: bool = True):
        self.M, self.ld, self.plane = M, ld, M * ld
        self.f = torch.zeros(M, ld, dtype=torch.float32, device=dev)
        self.s = torch.zeros(4, M, ld, dtype=torch.int16, device=dev) if split else None

    def sp(self, mask: int, ld: Optional[int] = None):
        """(base, ld, plane, mask) arguments for a producer kernel's split output."""
        if self.s is None or not mask:
            return (None, 0, 0, 0)
        return (self.s, ld if ld is not None else self.ld, self.plane, mask)


class View:
    """A column-offset view of a 2-D f32 buffer, passed to kernels as a raw pointer."""

    def __init__(self, t: torch.Tensor, col: int):
        self.t, self.col = t, col

    def data_ptr(self):
        return self.t.data_ptr() + self.col * self.t.element_size()

    def element_size(self):
        return self.t.element_size()


def _ptr(x):
    return x.data_ptr()
