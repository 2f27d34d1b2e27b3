"""DSV41 on the device: weight packing, per-slot caches and the row-batched forward pass.

One process per GPU.  ``forward(rows, ids)`` runs ``n <= max_rows`` rows (decode, multi-row
verify or a prefill chunk) through the 40 layers with the kernels of ``csrc/kernels/dsv41.cu``
plus the shared GEMV / tcgen05 GEMM, hyper-connection, argmax and all-reduce kernels.  Every
position-dependent quantity is read from device-resident row metadata, so a decode step is
replayable as one CUDA graph.

Tensor parallelism follows the reference's mapping (``crates/ferrite-models/src/dsv41/
weights.rs:27-330``): query heads / sinks / indexer heads by rank, ``wo_a`` by groups, ``wo_b``
by input columns (all-reduce #1), every routed expert on every rank with its intermediate dim
split (all-reduce #2), engram table by rows (all-reduce), indexer scores all-reduced; the
shared expert is split like the routed ones (the reference's ``DSV41_SHARED_TP`` mode) when
its slice stays a multiple of the quantisation block.

Dense e4m3 weights are expanded to bf16 at load time (exact: 4 significant bits times a power
of two) and stream through the bf16 tensor-core GEMV/GEMM; expert weights stay packed e2m1
with ue8m0 scales.  Replaces ``crates/ferrite-models/src/dsv41/chain_dev.rs`` (``DevChain``).
"""
from __future__ import annotations

import ctypes
from typing import Dict, List, Optional

import torch

from .. import _lib
from ..ops import quant as Q
from ..utils.switches import switches
from .dsv41_config import Dsv41Config
from .dsv41_engram import EngramLayout, hash_multipliers
from .dsv41_ref import rope_freqs
from .dsv41_weights import padded_inter, shard_tensor
from .glm import ROWMETA_BYTES, Act, GlmDeviceModel, RowSet, View

KMAXMIX = 24


class DictWeights:
    """Full f32 tensors by checkpoint name."""

    def __init__(self, weights: Dict[str, torch.Tensor]):
        self.w = weights

    def get(self, name: str) -> torch.Tensor:
        return self.w[name]

    def has(self, name: str) -> bool:
        return name in self.w


ATTN_MIN_PARTS = 1536   # (row, head, split) partials that the attention workspace always holds


def attn_splits(heads_local: int, n: int, sms: int = 148) -> int:
    """Key splits of the sparse attention for n rows: about one CTA per SM over (head tiles x rows x splits).  One
    decode row on a tensor-parallel shard takes 32 splits (4 clusters of 8 per head tile), 16 batched rows 4, a
    prefill chunk 1: a CTA holds 233 registers per thread, so only one is resident per SM and every further wave
    of CTAs costs a whole pass (16 rows at 16 splits: 60.7 us in 3.5 waves).  n * heads_local * splits never exceeds
    max(n * heads_local, ATTN_MIN_PARTS): the partial buffers are sized for that."""
    want = max(1, sms // (((heads_local + 7) // 8) * n))
    if want >= 32:
        return 32
    return want // 8 * 8 if want >= 8 else want   # multiples of 8 merge by clusters


class Dsv41DeviceModel:
    def __init__(self, cfg: Dsv41Config, src, rank: int = 0, world: int = 1, device="cuda", allreduce=None,
                 max_rows: int = 8, max_ctx: int = 1024, n_slots: int = 1, token_map=None):
        self.cfg, self.rank, self.world = cfg, rank, world
        self.dev = torch.device(device)
        self.K = _lib.lib()
        self.allreduce = allreduce
        assert world == 1 or allreduce is not None
        self.max_rows, self.max_ctx, self.n_slots = max_rows, max_ctx, n_slots
        assert cfg.hc_mult == 4 and cfg.n_heads % world == 0 and cfg.o_groups % world == 0
        assert cfg.index_n_heads % world == 0
        self.Hl = cfg.n_heads // world
        self.Gl = cfg.o_groups // world
        self.IHl = cfg.index_n_heads // world
        self.Il = padded_inter(cfg, world) if world > 1 else cfg.moe_inter_dim
        per = (cfg.moe_inter_dim + world - 1) // world
        self.shared_tp = world > 1 and per * world == cfg.moe_inter_dim
        self.Is_real = per if self.shared_tp else cfg.moe_inter_dim      # columns of the shared expert this rank owns
        self.Is = (self.Is_real + 63) // 64 * 64                        # zero-padded to the tensor-core GEMV's k-block
        self.tc_min_rows = switches().d4_tc_min_rows
        self.fused_rows = switches().d4_fused_rows
        from ..parallel.status import StatusArena
        self.arena = getattr(allreduce, "arena", None) or StatusArena(self.dev, 2048)
        self.tc_status = self.arena.status("tcgen05")
        self.row_status = self.arena.status("rows")
        self.tc_gemv_min_n = 0
        self.fp4_mma = switches().d4_fp4_mma   # tensor-core routed experts (decode rows)
        self.fp4_mma_rows = 1 << 30
        # row count from which the routed experts run as block-scaled tcgen05 grouped GEMMs (csrc/kernels/mx_gemm.cu):
        # below it the weight-streaming mma.sync kernels stream every (row, slot) pair's expert once per pair
        self.mx_min_rows = switches().d4_mx_min_rows
        self._mx_ws = None
        self._xq_ready = False
        # tensor-core sparse attention (head_dim 512), opt-in: at decode sizes (640 keys) it measured 21.6 us against
        # 16.3 us for the SIMT kernel with the in-kernel split merge (8 heads), and 2.37 vs 2.15 ms on the 8-layer bench
        self.attn_tc = switches().d4_attn_tc
        self._tc_part = None
        self._tc_ticket = None
        # GEMV + all-reduce + hyper-connection fold as one launch (csrc/kernels/gemv_ar.cu)
        self.fused = None
        if world > 1:
            self.fused = getattr(allreduce, "fused", None)
        else:
            from ..parallel.symm import FusedGemvAllReduce
            self.fused = FusedGemvAllReduce(self.dev, 0, 1, arena=self.arena)
        self._fold_next = None
        self._folded = False
        self._wide_ready = False   # the closing GEMV left mix-dot AND Gram partials: the column-parallel front can run
        self._part_stale = False   # the partial tile counts were consumed by a kernel that does not clear them
        self.debug_hook = None
        self.win_cap = cfg.window_size + max_rows
        # compressor ring: positions that one forward may look back over (ratio + rows of the forward)
        self.depth = max(16, max_rows + max([r for r in cfg.compress_ratios] + [1]))
        self.token_map = token_map
        self.layout = EngramLayout.from_config(cfg)
        self._pack(src)
        self._alloc()

    gemv = GlmDeviceModel.gemv

    # ---- packing -------------------------------------------------------------------------------
    def _bf(self, t):
        return t.to(self.dev, torch.bfloat16).contiguous()

    def _f(self, t):
        return t.to(self.dev, torch.float32).contiguous()

    def _sh(self, src, name):
        return shard_tensor(self.cfg, name, src.get(name), self.rank, self.world)

    def _pack_block(self, src, p: str, layer: int) -> dict:
        cfg = self.cfg
        a, f = p + "attn.", p + "ffn."
        L: dict = {"layer": layer, "ratio": cfg.ratio(layer)}
        L["w_qkv_a"] = self._bf(torch.cat([src.get(a + "wq_a.weight"), src.get(a + "wkv.weight")], 0))
        L["q_norm"] = self._f(src.get(a + "q_norm.weight"))
        L["kv_norm"] = self._f(src.get(a + "kv_norm.weight"))
        L["wq_b"] = self._bf(self._sh(src, a + "wq_b.weight"))
        L["sink"] = self._f(self._sh(src, a + "attn_sink"))
        L["wo_a"] = self._bf(self._sh(src, a + "wo_a.weight"))
        L["wo_b"] = self._bf(self._sh(src, a + "wo_b.weight"))
        if layer < cfg.n_layers and cfg.is_kv_source(layer):
            c = a + "compressor."
            ws = [src.get(c + "wkv.weight")]
            if cfg.ratio(layer) > 1:
                ws.append(src.get(c + "wgate.weight"))
            L["c_w"] = self._f(torch.cat(ws, 0))
            L["c_norm"] = self._f(src.get(c + "norm.weight"))
            L["i_wk"] = self._bf(src.get(a + "indexer.wk.weight"))
            L["i_knorm"] = self._f(src.get(a + "indexer.k_norm.weight"))
        if layer < cfg.n_layers and cfg.is_index_source(layer):
            L["i_wq_b"] = self._bf(self._sh(src, a + "indexer.wq_b.weight"))
            L["i_wproj"] = self._bf(self._sh(src, a + "indexer.weights_proj.weight"))
        L["attn_norm"] = self._f(src.get(p + "attn_norm.weight"))
        L["ffn_norm"] = self._f(src.get(p + "ffn_norm.weight"))
        for w in ("attn", "ffn"):
            L[f"hc_{w}_fn"] = self._f(src.get(p + f"hc_{w}_fn"))
            L[f"hc_{w}_base"] = self._f(src.get(p + f"hc_{w}_base"))
            L[f"hc_{w}_scale"] = self._f(src.get(p + f"hc_{w}_scale"))
        E, topk = cfg.moe_shape(layer)
        L["E"], L["topk"] = E, topk
        L["gate_w"] = self._bf(src.get(f + "gate.weight"))
        L["gate_b"] = self._f(src.get(f + "gate.bias"))
        L["gate_bvl"] = self._f(src.get(f + "gate.bias_vl")) if src.has(f + "gate.bias_vl") else None
        d, Il = cfg.dim, self.Il
        if hasattr(src, "expert_pack"):
            L["w13"], L["s13"], L["w2"], L["s2"] = src.expert_pack(f, E, Il, self.rank, self.world, self.dev)
        else:
            w13 = torch.empty(E, 2, Il, d // 2, dtype=torch.uint8, device=self.dev)
            s13 = torch.empty(E, 2, Il, d // 32, dtype=torch.uint8, device=self.dev)
            w2 = torch.empty(E, d, Il // 2, dtype=torch.uint8, device=self.dev)
            s2 = torch.empty(E, d, Il // 32, dtype=torch.uint8, device=self.dev)
            for e in range(E):
                for k, nm in enumerate(("w1", "w3")):
                    pk, sc = Q.quant_fp4_weight(self._sh(src, f + f"experts.{e}.{nm}.weight").float(), cfg.fp4_block)
                    w13[e, k].copy_(pk)
                    s13[e, k].copy_(sc)
                pk, sc = Q.quant_fp4_weight(self._sh(src, f + f"experts.{e}.w2.weight").float(), cfg.fp4_block)
                w2[e].copy_(pk)
                s2[e].copy_(sc)
            L["w13"], L["s13"], L["w2"], L["s2"] = w13, s13, w2, s2
        # tensor-core expert kernels want 128-value k-blocks and quad-interleaved weight bytes (repacked in place)
        L["fp4_mma"] = self.fp4_mma and d % 128 == 0 and Il % 64 == 0
        if L["fp4_mma"]:
            for t in (L["w13"], L["w2"]):
                self.K.call("fb_d4_fp4_repack", t, t.numel() // t.shape[-1], t.shape[-1], 0)
        # block-scaled tcgen05 path for prefill-sized row counts: weight scale bytes once more, in the layout tcgen05.cp
        # reads (1/16 of the weight bytes); the packed weights are shared with the decode kernels (either byte order)
        L["mx"] = (self.mx_min_rows > 0 and self.max_rows >= self.mx_min_rows and (2 * Il) % 128 == 0 and d % 128 == 0
                   and Il % 32 == 0 and E <= 512 and (not L["fp4_mma"] or Il % 64 == 0))
        if L["mx"]:
            from ..ops import mx
            L["sfa13"] = mx.pack_weight_scales(L["s13"].view(E, 2 * Il, d // 32))
            L["sfa2"] = mx.pack_weight_scales(L["s2"])
        sw1, sw3, sw2 = (src.get(f + f"shared_experts.{n}.weight") for n in ("w1", "w3", "w2"))
        if self.shared_tp:
            lo = self.rank * self.Is_real
            sw1, sw3, sw2 = sw1[lo:lo + self.Is_real], sw3[lo:lo + self.Is_real], sw2[:, lo:lo + self.Is_real]
        pad = self.Is - sw1.shape[0]
        if pad:   # padded channels compute silu(0) * 0 = 0 and meet zero columns of w2
            z = torch.zeros(pad, sw1.shape[1], dtype=sw1.dtype, device=sw1.device)
            sw1, sw3 = torch.cat([sw1, z], 0), torch.cat([sw3, z], 0)
            sw2 = torch.cat([sw2, torch.zeros(sw2.shape[0], pad, dtype=sw2.dtype, device=sw2.device)], 1)
        L["sh_w13"] = self._bf(torch.cat([sw1, sw3], 0))
        L["sh_w2"] = self._bf(sw2)
        return L

    def _pack(self, src):
        cfg = self.cfg
        self.embed = self._bf(src.get("embed.weight"))
        self.norm_w = self._f(src.get("norm.weight"))
        # vocab-sliced head when the collective carries a cross-rank argmax: each rank streams 1/world of the rows
        V = cfg.vocab_size
        self.xargmax = getattr(self.allreduce, "argmax", None) if self.world > 1 else None
        if self.xargmax is not None and V % self.world:
            self.xargmax = None
        self.Vl = V // self.world if self.xargmax is not None else V
        self.v_lo = self.rank * self.Vl if self.xargmax is not None else 0
        self.head = self._bf(src.get("head.weight")[self.v_lo:self.v_lo + self.Vl])
        self.layers: List[dict] = []
        for l in range(cfg.n_layers):
            p = f"layers.{l}."
            L = self._pack_block(src, p, l)
            ei = cfg.engram_index(l)
            if ei >= 0:
                rows = cfg.engram_num_embeddings[ei]
                per = (rows + self.world - 1) // self.world
                L["e_idx"] = ei
                L["e_lo"], L["e_hi"] = self.rank * per, min(rows, (self.rank + 1) * per)
                if hasattr(src, "engram_pack"):     # a source that hands the shard over in its device form
                    L["e_table"], L["e_scale"] = src.engram_pack(p, L["e_lo"], L["e_hi"], self.dev)
                else:
                    tab = self._sh(src, p + "engram.embed.weight").float()
                    q, sc = Q.fp8_act_quant(tab, cfg.fp8_block)
                    L["e_table"] = q.to(torch.float8_e4m3fn).view(torch.uint8).to(self.dev).contiguous()
                    L["e_scale"] = sc.to(self.dev).contiguous()
                L["e_wkv"] = self._bf(src.get(p + "engram.wkv.weight"))
                L["e_qk"] = self._f(src.get(p + "engram.q_weight").float() * src.get(p + "engram.k_weight").float())
            self.layers.append(L)
        self.mtp: List[dict] = []
        if cfg.dspark_block_size and cfg.n_mtp_layers and src.has("mtp.0.main_proj.weight"):
            for j in range(cfg.n_mtp_layers):
                self.mtp.append(self._pack_block(src, f"mtp.{j}.", cfg.n_layers + j))
            last = f"mtp.{cfg.n_mtp_layers - 1}."
            self.d_main_proj = self._bf(src.get("mtp.0.main_proj.weight"))
            self.d_main_norm = self._f(src.get("mtp.0.main_norm.weight"))
            self.d_norm = self._f(src.get(last + "norm.weight"))
            self.d_membed = self._bf(src.get(last + "markov_head.embed.weight"))
            self.d_mhead = self._bf(src.get(last + "markov_head.head.weight")[self.v_lo:self.v_lo + self.Vl])
            self.d_conf = self._f(src.get(last + "confidence_head.proj.weight"))
        self.freq_win = self._f(rope_freqs(cfg.rope_head_dim, cfg.rope_theta, 0, 1.0, cfg.beta_fast, cfg.beta_slow))
        self.freq_cmp = self._f(rope_freqs(cfg.rope_head_dim, cfg.compress_rope_theta, cfg.original_seq_len,
                                           cfg.rope_factor, cfg.beta_fast, cfg.beta_slow))
        if self.layout is not None:
            cv = cfg.engram_compressed_vocab_size
            tm = self.token_map if self.token_map is not None else [t % cv for t in range(cfg.vocab_size)]
            self.e_map = torch.tensor(list(tm), dtype=torch.int32, device=self.dev)
            self.e_pad = int(tm[cfg.engram_pad_id])
            self.e_mult = hash_multipliers(self.layout.layer_ids, self.layout.max_ngram, cv).to(self.dev).contiguous()
            self.e_primes = self.layout.flat_primes().to(self.dev).contiguous()
            self.e_offs = self.layout.offsets().to(self.dev).contiguous()

    # ---- buffers -------------------------------------------------------------------------------
    def _z(self, *shape, dtype=torch.float32):
        return torch.zeros(*shape, dtype=dtype, device=self.dev)

    def _alloc(self):
        cfg, M, S = self.cfg, self.max_rows, self.n_slots
        d, hd, ql = cfg.dim, cfg.head_dim, cfg.q_lora_rank
        ws: dict = {}
        ws["R0"], ws["R1"] = self._z(M, 4, d), self._z(M, 4, d)
        ws["R"] = ws["R0"]
        ws["hc_acc"] = self._z(M, KMAXMIX + 1)
        ws["pre0"], ws["pre1"] = self._z(M, 4), self._z(M, 4)
        ws["post"], ws["comb"] = self._z(M, 4), self._z(M, 16)
        ws["x"] = Act(self.dev, M, d)
        ws["xq"] = Act(self.dev, M, d)
        ws["qa"] = self._z(M, ql + hd)
        ws["qr"] = Act(self.dev, M, ql)
        ws["q"] = self._z(M, self.Hl * hd)
        ws["o"] = Act(self.dev, M, self.Hl * hd)
        ws["low"] = Act(self.dev, M, self.Gl * cfg.o_lora_rank)
        # split-K attention: keys of a row are spread over up to 16 CTAs per head tile
        lmax = cfg.window_size + cfg.index_topk + max(cfg.dspark_block_size, 1)
        self.at_split = max(1, min(16, (lmax + 31) // 32))
        # the split count follows the row count (`_attn_splits`): about one CTA per SM, at most 32 splits
        at_parts = max(M * self.Hl * self.at_split, ATTN_MIN_PARTS)
        ws["at_o"] = self._z(at_parts * hd)
        ws["at_ml"] = self._z(at_parts * 2)
        ws["at_ticket"] = self._z(M * ((self.Hl + 7) // 8), dtype=torch.int32)   # split-merge tickets (left at zero)
        ws["y"] = self._z(M, d)
        ws["ckv"] = self._z(M, 2 * hd)
        ws["lat"] = self._z(M, hd)
        ws["flag"] = self._z(M, dtype=torch.int32)
        ws["kraw"] = self._z(M, cfg.index_head_dim)
        ws["iq"] = self._z(M, self.IHl * cfg.index_head_dim)
        ws["iw"] = self._z(M, max(self.IHl, 8))
        self.ccap = {r: self.max_ctx // r for r in set(cfg.compress_ratios) if r > 0}
        cmax = max(self.ccap.values()) if self.ccap else 32
        ws["score"] = self._z(M, cmax)
        nbmax = (cmax + cfg.candidate_block_size - 1) // cfg.candidate_block_size
        ws["bscore"] = self._z(M, nbmax)
        ws["bidx"] = self._z(M, max(1, min(cfg.candidate_topk_blocks, nbmax)), dtype=torch.int32)
        ws["cand"] = self._z(M, cmax, dtype=torch.uint8)
        ws["topk"] = torch.full((M, cfg.index_topk), -1, dtype=torch.int32, device=self.dev)
        Emax = max(cfg.n_routed_experts, cfg.dspark_n_routed_experts)
        kmax = max(cfg.n_activated_experts, cfg.dspark_n_activated_experts)
        ws["rlogit"] = self._z(M, Emax)
        ws["ridx"] = self._z(M, kmax, dtype=torch.int32)
        ws["rw"] = self._z(M, kmax)
        ws["h"] = Act(self.dev, M * kmax, self.Il)
        ws["gu"] = self._z(M, 2 * self.Is)
        ws["hs"] = Act(self.dev, M, self.Is)
        ws["logits"] = self._z(M, cfg.vocab_size)
        ws["amax_part"] = self._z(M * 64, dtype=torch.int64)
        ws["out_ids"] = self._z(M, dtype=torch.int32)
        ws["mh"] = self._z(M, d * max(1, len(cfg.dspark_target_layer_ids)))
        ws["is_image"] = self._z(M, dtype=torch.uint8)
        if self.layout is not None:
            cols = self.layout.hash_cols
            ws["ehash"] = self._z(M, len(self.layout.layer_ids), cols, dtype=torch.int64)
            ws["egat"] = Act(self.dev, M, cols * cfg.engram_head_dim)
            ws["ekv"] = self._z(M, (cfg.hc_mult + 1) * d)
            self.e_hist = torch.full((S, self.max_ctx), -1, dtype=torch.int32, device=self.dev)
        if self.mtp:
            B, rk = cfg.dspark_block_size, cfg.dspark_markov_rank
            ws["mhq"] = Act(self.dev, M, ws["mh"].shape[1])
            ws["mx"] = Act(self.dev, M, d)
            ws["mkv"] = self._z(M, hd)
            ws["d_extra"] = self._z(M, hd)
            ws["d_ids"] = self._z(B, dtype=torch.int32)
            ws["d_out"] = self._z(B + 1, dtype=torch.int32)
            ws["d_me"] = Act(self.dev, 1, rk)
            ws["d_me_all"] = self._z(B, rk)
            ws["d_xc"] = self._z(M, d)
        self.ws = ws
        # per-slot caches
        nl = cfg.n_total_layers
        self.ring = torch.zeros(nl, S, self.win_cap, hd, dtype=torch.bfloat16, device=self.dev)
        self.comp: Dict[int, torch.Tensor] = {}
        self.kidx: Dict[int, torch.Tensor] = {}
        self.cring: Dict[int, tuple] = {}
        for l in cfg.kv_source_layers:
            cap = self.ccap[cfg.ratio(l)]
            self.comp[l] = torch.zeros(S, cap, hd, dtype=torch.bfloat16, device=self.dev)
            self.kidx[l] = torch.zeros(S, cap, cfg.index_head_dim, dtype=torch.bfloat16, device=self.dev)
            if cfg.ratio(l) > 1:
                self.cring[l] = (self._z(S, self.depth, hd), self._z(S, self.depth, hd))
        self.seq_len = self._z(S, dtype=torch.int32)

    def reset_slot(self, slot: int):
        self.seq_len[slot] = 0

    def make_rows(self, slots: List[int], gsizes: List[int]) -> RowSet:
        return GlmDeviceModel.make_rows(self, slots, gsizes)

    # ---- sequence snapshots (host-side prefix cache, speculative experiments) ------------------
    def snapshot_slot(self, slot: int = 0) -> dict:
        """Everything a sequence owns, copied to host memory (reference: the host-snapshot KV prefix
        cache of ``crates/ferrite-dsv41/src/serve.rs:79-101,934-1020``)."""
        n = int(self.seq_len[slot])
        snap = {"len": n, "ring": self.ring[:, slot].cpu()}
        for l, t in self.comp.items():
            used = (n // self.cfg.ratio(l)) + 1
            snap[f"comp{l}"] = t[slot, :used].cpu()
            snap[f"kidx{l}"] = self.kidx[l][slot, :used].cpu()
        for l, (a, b) in self.cring.items():
            snap[f"cring{l}"] = (a[slot].cpu(), b[slot].cpu())
        if self.layout is not None:
            snap["e_hist"] = self.e_hist[slot, :n].cpu()
        return snap

    def restore_slot(self, snap: dict, slot: int = 0) -> None:
        n = snap["len"]
        self.ring[:, slot].copy_(snap["ring"])
        for l, t in self.comp.items():
            used = snap[f"comp{l}"].shape[0]
            t[slot, :used].copy_(snap[f"comp{l}"])
            self.kidx[l][slot, :used].copy_(snap[f"kidx{l}"])
        for l, (a, b) in self.cring.items():
            a[slot].copy_(snap[f"cring{l}"][0])
            b[slot].copy_(snap[f"cring{l}"][1])
        if self.layout is not None:
            self.e_hist[slot, :n].copy_(snap["e_hist"])
        self.seq_len[slot] = n

    # ---- forward ---------------------------------------------------------------------------------
    def _reduce(self, t, n):
        if self.world > 1:
            step = max(1, getattr(self.allreduce, "max_elems", t[:n].numel()) // t.shape[1])
            for r0 in range(0, n, step):   # the one-shot all-reduce takes a bounded payload per launch
                self.allreduce(t[r0:min(n, r0 + step)])

    def _argmax(self, logits, out_ids, n):
        """Greedy ids of `n` rows of logits [n, Vl] (this rank's vocab slice when the head is sliced: the
        partial keys are merged across the ranks and every rank gets the global id)."""
        ws = self.ws
        if self.xargmax is None:
            self.K.call("fb_argmax", logits, self.Vl, ws["amax_part"], out_ids, None, n, self.Vl, 1, 0)
        else:
            self.xargmax(logits, self.Vl, ws["amax_part"], n, self.Vl, self.v_lo, out_ids)

    def _quant(self, src_f, dst: Act, n, K, ld=None, mask=1):
        """dst.f / dst planes = e4m3-per-32 round trip of src (may alias dst.f); mask 1: bf16 planes,
        2: f16 planes, 3: both."""
        ld = ld if ld is not None else dst.ld
        self.K.call("fb_d4_quant_rows", src_f, ld, dst.f, dst.ld, n, K, *dst.sp(mask))

    def _hc_post_mix(self, fn_next, n, first=False):
        cfg, ws = self.cfg, self.ws
        if self._folded:   # the sublayer's last GEMV already did hc_post and the mix dots
            self._folded = False
            return
        rin = ws["R"]
        mix = (2 + cfg.hc_mult) * cfg.hc_mult
        if first:
            self.K.call("fb_hc_post_mix", rin, rin, None, None, None, fn_next, ws["hc_acc"], n, cfg.dim, mix)
            return
        rout = ws["R1"] if rin is ws["R0"] else ws["R0"]
        self.K.call("fb_hc_post_mix", rin, rout, ws["y"], ws["post"], ws["comb"], fn_next, ws["hc_acc"], n, cfg.dim, mix)
        ws["R"] = rout

    def _out_gemv(self, w, x: Act, n, N, K, accumulate=False):
        """Last GEMV of a sublayer into ws['y'], summed over ranks; inside a hyper-connection site
        the fused kernel also applies hc_post and leaves the next site's mix-dot partials."""
        ws = self.ws
        fold, self._fold_next = self._fold_next, None
        ok = (self.fused is not None and x.s is not None and n <= self.fused_rows and K % 64 == 0 and x.ld % 8 == 0 and N % 32 == 0
              and (self.world == 1 or min(n, 8) * N <= self.fused.max_elems)   # the launcher walks 8-row windows
              and (self.world > 1 or fold is not None))
        if not ok:
            gar = getattr(self.allreduce, "gemm_fused", None) if self.world > 1 else None
            if (gar is not None and x.s is not None and n >= self.tc_min_rows and K % 8 == 0 and x.ld % 8 == 0
                    and ws["y"].shape[1] % 4 == 0 and gar.fits(n, N)):
                # prefill rows: TMA + tcgen05 GEMM with the two-shot all-reduce in its epilogue (one launch)
                gar(w, x.s, x.ld, ws["y"], ws["y"].shape[1], n, N, K, accumulate)
                return
            self.gemv(w, x, ws["y"], n, N, K, accumulate=accumulate)
            self._reduce(ws["y"], n)
            return
        f = None
        want_gram = False
        if fold is not None:
            rin = ws["R"]
            rout = ws["R1"] if rin is ws["R0"] else ws["R0"]
            f = (rin, rout, ws["post"], ws["comb"], fold[0], ws["hc_acc"], (2 + self.cfg.hc_mult) * self.cfg.hc_mult)
            ws["R"] = rout
            self._folded = True
            self._part_stale = False   # this launch rewrites the tile counts
            if fold[0] is not None and self.hc_wide and n <= 8 and N == self.cfg.dim and N // 16 <= 512 and N % 32 == 0:
                self._wide_ready = want_gram = True
        self.fused(w, None, x.s, x.ld, x.plane, ws["y"], N, n, N, K, accumulate, fold is None or self.debug is not None, f,
                   gram=want_gram)

    # hc_pre can also emit the e4m3 round trip of its output (two launches fewer per layer).  Off by default: measured
    # 1 % SLOWER at TP1 and on the TP8 shard (2.175 vs 2.161 ms, 5.94 vs 5.88 ms): hc_pre is a one-CTA latency chain
    # on the critical path, the separate quantiser spreads over many CTAs
    fuse_quant = property(lambda self: switches().d4_fuse_quant)
    moe_paired = True   # decode rows: router and shared-expert chains share their launches
    # decode rows: the front as a column-parallel kernel fed by the closing GEMV's Gram partials (it also quantises)
    hc_wide = property(lambda self: switches().hc_pre_wide and self.cfg.hc_mult == 4)

    def _hc_pre(self, L, site, ln, n, coeffs=True, quant=True):
        """Coefficients of this site (stored for the next one) and the contraction with the previous
        site's `pre`; leaves the normed input in ws['x'] (f32 + bf16 planes).  When the closing GEMV of the previous
        sublayer left mix-dot and Gram partials (decode rows), the column-parallel kernel runs and also leaves the
        e4m3 round trip of x in ws['xq']."""
        quant = quant and self.fuse_quant
        cfg, ws = self.cfg, self.ws
        x = ws["x"]
        pin, pout = ws["pre_cur"], ws["pre_nxt"]
        if self._wide_ready:
            self._wide_ready = False
            assert coeffs and n <= 8
            part, gram, part_n, ld = self.fused.wide_partials()
            xq = ws["xq"]
            self.K.call("fb_hc_pre_wide_offset", ws["R"], part, gram, part_n, ld, L[f"hc_{site}_scale"],
                        L[f"hc_{site}_base"], ln, pin, pout, x.f, ws["post"], ws["comb"], n, cfg.dim,
                        (2 + cfg.hc_mult) * cfg.hc_mult, float(cfg.norm_eps), float(cfg.hc_eps), cfg.hc_sinkhorn_iters,
                        *x.sp(1), xq.f, *xq.sp(3))
            self._xq_ready = True
            self._part_stale = True
            ws["pre_cur"], ws["pre_nxt"] = pout, pin
            return
        if self._part_stale:   # no launch rewrote the tile counts since the column-parallel front read them
            self._part_stale = False
            self.fused.part_n.zero_()
        self.K.call("fb_d4_hc_pre", ws["R"], ws["hc_acc"] if coeffs else None,
                    L[f"hc_{site}_scale"] if coeffs else None, L[f"hc_{site}_base"] if coeffs else None, ln, pin, pout,
                    ws["post"], ws["comb"], x.f, None, n, cfg.dim, cfg.hc_mult, float(cfg.norm_eps), float(cfg.hc_eps),
                    cfg.hc_sinkhorn_iters, *x.sp(1),
                    *(self.fused.partials() if self.fused is not None and coeffs and n <= self.fused_rows else (None, None, 0)),
                    *((ws["xq"].f, *ws["xq"].sp(3)) if quant else (None, None, 0, 0, 0)))
        self._xq_ready = quant   # the sublayer's first quantisation of x is already done
        if coeffs:
            ws["pre_cur"], ws["pre_nxt"] = pout, pin

    def _attn_splits(self, n: int) -> int:
        return attn_splits(self.Hl, n)

    def _attention(self, L, rs: RowSet, shared: dict, ring, extra=None, n_extra=0, win_mode=0):
        cfg, ws, n = self.cfg, self.ws, rs.n
        d, hd, ql, rd = cfg.dim, cfg.head_dim, cfg.q_lora_rank, cfg.rope_head_dim
        layer, r = L["layer"], L["ratio"]
        x, xq, qr = ws["x"], ws["xq"], ws["qr"]
        freqs = self.freq_cmp if r > 0 else self.freq_win
        if not self._xq_ready:
            self._quant(x.f, xq, n, d)
        self._xq_ready = False
        self.gemv(L["w_qkv_a"], xq, ws["qa"], n, ql + hd, d)
        # one launch for both consumers of the q-lora | kv row: q-lora norm + quantiser, kv norm + rope + quantiser + store
        # (a draft block's own KV rows stay out of the ring: they go to `extra`)
        self.K.call("fb_d4_qnorm_kv_append", ws["qa"], ql + hd, ql, L["q_norm"], qr.f, ql, float(cfg.norm_eps), *qr.sp(1),
                    L["kv_norm"], freqs, rs.meta, ring if extra is None else None, self.win_cap, extra, n, hd, rd, 0)
        self.gemv(L["wq_b"], qr, ws["q"], n, self.Hl * hd, ql)
        comp, idx, ktop, ccap = None, None, 0, 0
        if r > 0:
            src = cfg.kv_source_of(layer)
            ccap = self.ccap[r]
            if "c_w" in L:
                nc = L["c_w"].shape[0]
                for r0 in range(0, n, 8):   # the f32-weight GEMV takes 8 rows per launch
                    self.K.call("fb_d4_gemv_f32w", L["c_w"], View(x.f, r0 * x.f.shape[1]), d, View(ws["ckv"], r0 * 2 * hd),
                                2 * hd, min(8, n - r0), nc, d)
                rk, rsc = self.cring.get(layer, (None, None))
                self.K.call("fb_d4_compress", ws["ckv"], View(ws["ckv"], hd), 2 * hd, rs.meta, rk, rsc, self.depth,
                            L["c_norm"], ws["lat"], ws["flag"], n, hd, r, float(cfg.norm_eps))
                self.gemv(L["i_wk"], ws["lat"], ws["kraw"], n, cfg.index_head_dim, hd)
                self.K.call("fb_d4_index_k_store", ws["kraw"], cfg.index_head_dim, ws["flag"], rs.meta, L["i_knorm"], freqs,
                            self.kidx[layer], ccap, n, cfg.index_head_dim, rd, r, float(cfg.norm_eps))
                self.K.call("fb_d4_latent_store", ws["lat"], ws["flag"], rs.meta, freqs, self.comp[layer], ccap, n, hd, rd, r)
            if "i_wq_b" in L:
                ID = cfg.index_head_dim
                self.gemv(L["i_wq_b"], qr, ws["iq"], n, self.IHl * ID, ql)
                self.K.call("fb_d4_rope_heads", ws["iq"], self.IHl * ID, n, self.IHl, ID, rd, freqs, rs.meta, 0, 0, 1,
                            None, 0, 0, 0)
                self.gemv(L["i_wproj"], x, ws["iw"], n, self.IHl, d, ldo=ws["iw"].shape[1])
                lds = ws["score"].shape[1]
                self.K.call("fb_d4_index_score", ws["iq"], self.IHl * ID, ws["iw"], ws["iw"].shape[1], self.kidx[src], ccap,
                            rs.meta, ws["score"], lds, n, self.IHl, ID, r, float(ID ** -0.5 * cfg.index_n_heads ** -0.5))
                self._reduce(ws["score"], n)
                mask, ldm = None, 0
                if layer == cfg.candidate_source_layer:
                    bs = cfg.candidate_block_size
                    ldb = ws["bscore"].shape[1]
                    kb = ws["bidx"].shape[1]
                    self.K.call("fb_d4_block_max", ws["score"], lds, rs.meta, r, bs, ws["bscore"], ldb, n)
                    self.K.call("fb_d4_topk_sorted", ws["bscore"], ldb, None, 0, rs.meta, r, bs, kb, ws["bidx"], kb, n)
                    self.K.call("fb_d4_cand_mask", ws["bidx"], kb, kb, bs, ws["cand"], ws["cand"].shape[1], n)
                elif cfg.uses_candidates(layer):
                    mask, ldm = ws["cand"], ws["cand"].shape[1]
                self.K.call("fb_d4_topk_sorted", ws["score"], lds, mask, ldm, rs.meta, r, 1, cfg.index_topk, ws["topk"],
                            cfg.index_topk, n)
            comp, idx, ktop = self.comp[src], ws["topk"], cfg.index_topk
        o = ws["o"]
        if self.attn_tc and hd == 512 and extra is None and self.Hl <= 64:
            # tensor cores: all heads of a row share one key sequence, so QK^T and PV are two small GEMMs per 64-key tile
            nsp = min(self.at_split, (cfg.window_size + (ktop if idx is not None else 0) + 63) // 64)
            self.K.call("fb_d4_sparse_attn_tc", ws["q"], self.Hl * hd, ring, self.win_cap, cfg.window_size, comp, ccap, idx,
                        cfg.index_topk, ktop, L["sink"], freqs, rd, rs.meta, 0, win_mode, float(hd ** -0.5), self.Hl,
                        o.f, self.Hl * hd, n, max(1, nsp), ws["at_o"], ws["at_ml"], *o.sp(1))
        else:
            self.K.call("fb_d4_sparse_attn", ws["q"], self.Hl * hd, ring, self.win_cap, cfg.window_size, comp, ccap, idx,
                        cfg.index_topk, ktop, extra, n_extra, L["sink"], freqs, rd, rs.meta, 0, win_mode, float(hd ** -0.5),
                        self.Hl, hd, o.f, self.Hl * hd, n, self._attn_splits(n),
                        ws["at_o"], ws["at_ml"], *o.sp(1), ws["at_ticket"])
        low = ws["low"]
        R_ = cfg.o_lora_rank
        self.gemv(L["wo_a"], o, low, n, self.Gl * R_, cfg.heads_per_group * hd, ldx=self.Hl * hd, group_rows=R_)
        self._quant(low.f, low, n, self.Gl * R_)
        self._out_gemv(L["wo_b"], low, n, d, self.Gl * R_)

    def _moe_mx(self, L, n):
        """Routed experts of `n` rows as two block-scaled tcgen05 grouped GEMMs: pairs sorted by expert, rows
        quantised (e4m3 + ue8m0 per 32) straight into their sorted places, gate | up GEMM, weighted SwiGLU +
        requantisation, down GEMM, slot-ordered combine into ws['y'].  Every expert's weights stream once per
        call, however many rows it has."""
        from ..ops import mx
        cfg, ws, K = self.cfg, self.ws, self.K
        d, Il, E, topk = cfg.dim, self.Il, L["E"], L["topk"]
        npairs = n * topk
        W = self._mx_ws
        if W is None:
            M, kmax = self.max_rows, ws["ridx"].shape[1]
            P = M * kmax
            i32 = lambda *s_: torch.zeros(*s_, dtype=torch.int32, device=self.dev)
            u8 = lambda *s_: torch.zeros(*s_, dtype=torch.uint8, device=self.dev)
            W = self._mx_ws = {
                "pos": i32(P), "wts": self._z(P), "counts": i32(512), "offsets": i32(513),
                "tiles": i32(512 + P // 32 + 1, 4), "n_tiles": i32(1),
                "x8": u8(P, d), "xsf": u8(P, mx.sf_ld(d)), "h": self._z(P, 2 * Il), "a8": u8(P, Il),
                "asf": u8(P, mx.sf_ld(Il)), "ypair": self._z(P, d)}
        bn = mx.pick_bn(max(1.0, npairs / E))
        K.call("fb_mx_sort", ws["ridx"], ws["rw"], npairs, 0, E, bn, W["pos"], W["wts"], W["counts"], W["offsets"], W["tiles"],
               W["n_tiles"], W["tiles"].shape[0])
        K.call("fb_mx_quant_scatter", ws["x"].f, ws["x"].ld, W["pos"], topk, n, d, W["x8"], W["xsf"], W["xsf"].shape[1])
        quad = bool(L["fp4_mma"])
        mx.mx_gemm_grouped(L["w13"].view(E, 2 * Il, d // 2), L["sfa13"], W["x8"][:npairs], W["xsf"], W["tiles"], W["n_tiles"],
                           W["h"], bn, self.tc_status, quad=quad, m_total=npairs)
        lim = float(cfg.swiglu_limit) if cfg.swiglu_limit > 0 else 3.0e38
        K.call("fb_mx_swiglu_quant", W["h"], 2 * Il, W["wts"], View(W["offsets"], E), npairs, Il, lim, W["a8"], W["asf"],
               W["asf"].shape[1])
        mx.mx_gemm_grouped(L["w2"], L["sfa2"], W["a8"][:npairs], W["asf"], W["tiles"], W["n_tiles"], W["ypair"], bn,
                           self.tc_status, quad=quad, m_total=npairs)
        K.call("fb_mx_combine", W["ypair"], d, W["pos"], topk, ws["y"], ws["y"].shape[1], n, d, 0)

    def _moe(self, L, n):
        cfg, ws = self.cfg, self.ws
        d, x, xq = cfg.dim, ws["x"], ws["xq"]
        E, topk = L["E"], L["topk"]
        ldl = ws["rlogit"].shape[1]
        if (L["fp4_mma"] and n <= self.fp4_mma_rows and not (L.get("mx") and n >= self.mx_min_rows) and E <= 384
                and topk <= 32 and d % 64 == 0 and x.s is not None and xq.s is not None and self.moe_paired):
            # Decode rows.  The router chain (logits -> route) and the shared expert's chain (gate | up -> SwiGLU) do
            # not depend on each other: they share their launches (one two-problem GEMV, one route + SwiGLU kernel)
            if not self._xq_ready:
                self._quant(x.f, xq, n, d, mask=3)
            self._xq_ready = False
            hs, gu = ws["hs"], ws["gu"]
            self.K.call("fb_gemv_mma_bf16_dual", L["gate_w"], x.s, x.ld, x.plane, ws["rlogit"], ldl, E, d,
                        L["sh_w13"], xq.s, xq.ld, xq.plane, gu, gu.shape[1], 2 * self.Is, d, n)
            self.K.call("fb_d4_route_swiglu", ws["rlogit"], ldl, L["gate_b"], L["gate_bvl"],
                        ws["is_image"] if L["gate_bvl"] is not None else None, n, E, topk, float(cfg.route_scale),
                        ws["ridx"], ws["rw"], gu, gu.shape[1], hs.f, self.Is, self.Is, float(cfg.swiglu_limit), *hs.sp(1))
            h = ws["h"]
            f16 = lambda a: _lib.ctypes.c_void_p(a.s.data_ptr() + 4 * a.plane)   # plane 2 of the int16 planes
            self.K.call("fb_d4_expert_gate_up_mma", f16(xq), xq.ld, ws["ridx"], ws["rw"], L["w13"], L["s13"], h.f, n, topk,
                        self.Il, d, float(cfg.swiglu_limit))
            self.K.call("fb_d4_quant_rows", h.f, self.Il, h.f, self.Il, n * topk, self.Il, *h.sp(2))
            self.K.call("fb_d4_expert_down_mma", f16(h), ws["ridx"], L["w2"], L["s2"], ws["y"], d, n, topk, self.Il, d, 0)
            if not self.shared_tp:
                self._reduce(ws["y"], n)
            if self.shared_tp or self.world == 1:
                self._out_gemv(L["sh_w2"], hs, n, d, self.Is, accumulate=True)
            else:
                self._fold_next = None
                self.gemv(L["sh_w2"], hs, ws["y"], n, d, self.Is, accumulate=True)
            return
        self.gemv(L["gate_w"], x, ws["rlogit"], n, E, d, ldo=ldl)
        self.K.call("fb_d4_route", ws["rlogit"], ldl, L["gate_b"], L["gate_bvl"], ws["is_image"] if L["gate_bvl"] is not None else None,
                    n, E, topk, float(cfg.route_scale), ws["ridx"], ws["rw"])
        h = ws["h"]
        if L.get("mx") and n >= self.mx_min_rows:
            if not self._xq_ready:      # the shared expert below reads the quantised planes
                self._quant(x.f, xq, n, d)
            self._xq_ready = False
            self._moe_mx(L, n)
        elif L["fp4_mma"] and n <= self.fp4_mma_rows:
            # decode rows: e2m1 weights x f16 activations on the tensor cores (activations are e4m3 round trips,
            # exact in f16), one (row, slot) pair per CTA column
            if not self._xq_ready:
                self._quant(x.f, xq, n, d, mask=3)
            self._xq_ready = False
            f16 = lambda a: _lib.ctypes.c_void_p(a.s.data_ptr() + 4 * a.plane)   # plane 2 of the int16 planes
            self.K.call("fb_d4_expert_gate_up_mma", f16(xq), xq.ld, ws["ridx"], ws["rw"], L["w13"], L["s13"], h.f, n, topk,
                        self.Il, d, float(cfg.swiglu_limit))
            # (fb_d4_expert_down_mma_f32 quantises h while loading it and saves this launch, but every one of its
            # D / 16 CTAs then repeats the quantiser: 10.6 us against 1.7 + 7.2 us measured on the TP=4 shard)
            self.K.call("fb_d4_quant_rows", h.f, self.Il, h.f, self.Il, n * topk, self.Il, *h.sp(2))
            self.K.call("fb_d4_expert_down_mma", f16(h), ws["ridx"], L["w2"], L["s2"], ws["y"], d, n, topk, self.Il, d, 0)
        else:
            assert not L["fp4_mma"], "quad-interleaved expert weights need the tensor-core kernels"
            if not self._xq_ready:
                self._quant(x.f, xq, n, d)
            self._xq_ready = False
            self.K.call("fb_d4_expert_gate_up", xq.f, d, ws["ridx"], ws["rw"], L["w13"], L["s13"], h.f, n, topk, self.Il, d,
                        float(cfg.swiglu_limit))
            self.K.call("fb_d4_quant_rows", h.f, self.Il, h.f, self.Il, n * topk, self.Il, None, 0, 0, 0)
            self.K.call("fb_d4_expert_down", h.f, ws["ridx"], L["w2"], L["s2"], ws["y"], d, n, topk, self.Il, d, 0)
        if not self.shared_tp:
            self._reduce(ws["y"], n)
        hs = ws["hs"]
        self.gemv(L["sh_w13"], xq, ws["gu"], n, 2 * self.Is, d)
        # clamped SwiGLU and its e4m3-per-32 round trip in one launch
        self.K.call("fb_d4_swiglu_clamp_quant", ws["gu"], 2 * self.Is, hs.f, self.Is, n, self.Is, float(cfg.swiglu_limit),
                    *hs.sp(1))
        if self.shared_tp or self.world == 1:
            self._out_gemv(L["sh_w2"], hs, n, d, self.Is, accumulate=True)
        else:
            self._fold_next = None
            self.gemv(L["sh_w2"], hs, ws["y"], n, d, self.Is, accumulate=True)

    def _engram(self, L, rs, n):
        cfg, ws = self.cfg, self.ws
        lay = self.layout
        g = ws["egat"]
        cols, ehd = lay.hash_cols, cfg.engram_head_dim
        self.K.call("fb_d4_engram_gather", ws["ehash"], len(lay.layer_ids), L["e_idx"], cols, L["e_table"], L["e_scale"],
                    L["e_lo"], L["e_hi"], ehd, g.f, n)
        self._reduce(g.f, n)
        self._quant(g.f, g, n, cols * ehd)
        self.gemv(L["e_wkv"], g, ws["ekv"], n, (cfg.hc_mult + 1) * cfg.dim, cols * ehd)
        self.K.call("fb_d4_engram_apply", ws["R"], ws["ekv"], L["e_qk"], ws["is_image"] if self.has_images else None, n,
                    cfg.hc_mult, cfg.dim, float(cfg.norm_eps))

    has_images = False
    debug = None   # callable(name, tensor) for op-by-op comparison against the golden model's trace

    def _dbg(self, name, t):
        if self.debug is not None:
            self.debug(name, t)

    def forward(self, rs: RowSet, ids: torch.Tensor, advance: bool = True, want_logits: bool = True,
                image_embeds: Optional[torch.Tensor] = None, is_image: Optional[torch.Tensor] = None):
        """Run rs.n rows; ids [n] int32 on the device.  Leaves logits in ws['logits'], greedy ids in
        ws['out_ids'] and the DSpark target hiddens in ws['mh'].  Rows flagged in `is_image` [n] take
        their embedding from `image_embeds` [n, dim] (vision tower output), get no engram
        contribution and route with the image bias."""
        cfg, ws, n = self.cfg, self.ws, rs.n
        d = cfg.dim
        self.K.call("fb_prep_rows", rs.row_slot, rs.row_off, rs.row_gsize, self.seq_len, rs.meta, n, self.max_ctx,
                    self.row_status)
        ws["R"] = ws["R0"]
        self.K.call("fb_embed_expand", ids, self.embed, ws["R"], n, d, cfg.hc_mult, cfg.vocab_size)
        self.has_images = image_embeds is not None
        if self.has_images:
            mask = is_image.to(self.dev).bool()
            ws["is_image"][:n].copy_(mask)
            ws["R"][:n] = torch.where(mask[:, None, None], image_embeds.to(self.dev).float()[:, None, :], ws["R"][:n])
        else:
            ws["is_image"].zero_()
        ws["pre0"].zero_()
        ws["pre0"][:, 0] = 1.0
        ws["pre_cur"], ws["pre_nxt"] = ws["pre0"], ws["pre1"]
        if self.layout is not None:
            lay = self.layout
            self.K.call("fb_d4_engram_hash", ids, ws["is_image"] if self.has_images else None, rs.meta, self.e_map,
                        self.e_hist, self.max_ctx, self.e_mult, self.e_primes, self.e_offs, self.e_pad, n,
                        len(lay.layer_ids), lay.max_ngram, lay.n_heads, ws["ehash"])
        shared: dict = {}
        tgt = list(cfg.dspark_target_layer_ids)
        pending_mix = True   # the mix dots of the first site are not computed yet
        for l, L in enumerate(self.layers):
            if "e_idx" in L:
                self._engram(L, rs, n)
                pending_mix = True
            if l in tgt:
                self.K.call("fb_d4_copy_mean", ws["R"], ws["mh"], ws["mh"].shape[1], tgt.index(l) * d, n, cfg.hc_mult, d)
            if pending_mix:
                ws["hc_acc"].zero_()
                self._hc_post_mix(L["hc_attn_fn"], n, first=True)
                pending_mix = False
            self._hc_pre(L, "attn", L["attn_norm"], n)
            self._dbg(f"layers.{l}.attn_in", ws["x"].f[:n])
            self._fold_next = (L["hc_ffn_fn"],)
            self._attention(L, rs, shared, self.ring[l])
            self._dbg(f"layers.{l}.attn_o", ws["o"].f[:n])
            if L["ratio"] > 0:
                self._dbg(f"layers.{l}.topk", ws["topk"][:n])
            self._dbg(f"layers.{l}.attn_out", ws["y"][:n])
            self._hc_post_mix(L["hc_ffn_fn"], n)
            self._hc_pre(L, "ffn", L["ffn_norm"], n)
            nxt = self.layers[l + 1] if l + 1 < len(self.layers) else None
            fn_next = nxt["hc_attn_fn"] if nxt is not None and "e_idx" not in nxt else None
            self._fold_next = (fn_next,)
            self._moe(L, n)
            self._dbg(f"layers.{l}.route_idx", ws["ridx"][:n, :L["topk"]])
            self._dbg(f"layers.{l}.ffn_out", ws["y"][:n])
            self._hc_post_mix(fn_next, n)
            if fn_next is None:
                pending_mix = True
            self._dbg(f"layers.{l}.h", ws["R"][:n])
        self._hc_pre({}, "", self.norm_w, n, coeffs=False, quant=False)
        if want_logits:
            self.gemv(self.head, ws["x"], ws["logits"], n, self.Vl, d)
            self._argmax(ws["logits"], ws["out_ids"], n)
        if advance:
            self.K.call("fb_advance_rows", rs.meta, None, self.seq_len, n)

    # ---- DSpark (block draft over the main model's KV) ---------------------------------------------
    def dspark_seed(self, rs: RowSet, row0: int = 0, n: Optional[int] = None):
        """Write the main-model KV of rows row0..row0+n-1 of the last forward (their target-layer
        hiddens are in ws['mh']) into every DSpark layer's ring at those rows' positions.  `rs`
        must be the row set of that forward, with its metadata still valid."""
        cfg, ws = self.cfg, self.ws
        n = rs.n if n is None else n
        d, hd = cfg.dim, cfg.head_dim
        km = ws["mh"].shape[1]
        mh = ws["mh"][row0:]
        mhq, mx = ws["mhq"], ws["mx"]
        meta = View(rs.meta, row0 * ROWMETA_BYTES)
        self.K.call("fb_d4_quant_rows", mh, km, mhq.f, km, n, km, *mhq.sp(1))
        self.gemv(self.d_main_proj, mhq, mx, n, d, km)
        self.K.call("fb_rmsnorm", mx.f, None, None, self.d_main_norm, mx.f, n, d, d, d, float(cfg.norm_eps), None, 0, 0, 0)
        self._quant(mx.f, mx, n, d)
        for j, L in enumerate(self.mtp):
            # only the wkv rows of the fused [wq_a ; wkv] matrix
            wkv = View(L["w_qkv_a"], cfg.q_lora_rank * d)
            self.gemv(wkv, mx, ws["mkv"], n, hd, d)
            self.K.call("fb_d4_kv_append", ws["mkv"], hd, L["kv_norm"], self.freq_win, meta, self.ring[cfg.n_layers + j],
                        self.win_cap, None, n, hd, cfg.rope_head_dim, float(cfg.norm_eps), 0)

    def dspark_draft(self, rs_block: RowSet, t0: torch.Tensor):
        """Draft block after the committed sequence (seq_len rows, main KV seeded).  `t0` is a device
        int32 tensor [1] holding the last emitted token.  Leaves [t0, d1..dB] in ws['d_out'] and the
        block logits in ws['logits'][:B]."""
        cfg, ws = self.cfg, self.ws
        B, d = cfg.dspark_block_size, cfg.dim
        assert rs_block.n == B
        ids = ws["d_ids"]
        ids.fill_(cfg.dspark_noise_token_id)
        ids[0:1].copy_(t0)
        self.K.call("fb_prep_rows", rs_block.row_slot, rs_block.row_off, rs_block.row_gsize, self.seq_len, rs_block.meta, B,
                    self.max_ctx, self.row_status)
        ws["R"] = ws["R0"]
        self.K.call("fb_embed_expand", ids, self.embed, ws["R"], B, d, cfg.hc_mult, cfg.vocab_size)
        ws["pre0"].zero_()
        ws["pre0"][:, 0] = 1.0
        ws["pre_cur"], ws["pre_nxt"] = ws["pre0"], ws["pre1"]
        ws["hc_acc"].zero_()
        for j, L in enumerate(self.mtp):
            if j == 0:
                self._hc_post_mix(L["hc_attn_fn"], B, first=True)
            self._hc_pre(L, "attn", L["attn_norm"], B)
            self._fold_next = (L["hc_ffn_fn"],)
            self._attention(L, rs_block, {}, self.ring[cfg.n_layers + j], extra=ws["d_extra"], n_extra=B, win_mode=1)
            self._hc_post_mix(L["hc_ffn_fn"], B)
            self._hc_pre(L, "ffn", L["ffn_norm"], B)
            nxt = self.mtp[j + 1] if j + 1 < len(self.mtp) else None
            fn_next = nxt["hc_attn_fn"] if nxt else None
            self._fold_next = (fn_next,)
            self._moe(L, B)
            self._hc_post_mix(fn_next, B)
        x = ws["x"]
        self.K.call("fb_d4_hc_pre", ws["R"], None, None, None, self.d_norm, ws["pre_cur"], ws["pre_nxt"], ws["post"],
                    ws["comb"], x.f, ws["d_xc"], B, d, cfg.hc_mult, float(cfg.norm_eps), float(cfg.hc_eps),
                    cfg.hc_sinkhorn_iters, *x.sp(1), None, None, 0, None, None, 0, 0, 0)
        V, Vl, rk = cfg.vocab_size, self.Vl, cfg.dspark_markov_rank
        self.gemv(self.head, x, ws["logits"], B, Vl, d)
        out, me = ws["d_out"], ws["d_me"]
        out[0:1].copy_(t0)
        for i in range(B):
            self.K.call("fb_d4_gather_row", self.d_membed, View(out, i), rk, V, me.f, *me.sp(1))
            ws["d_me_all"][i].copy_(me.f[0])
            self.gemv(self.d_mhead, me, View(ws["logits"], i * Vl), 1, Vl, rk, accumulate=True)
            self._argmax(View(ws["logits"], i * Vl), View(out, i + 1), 1)
        return out

    def dspark_confidence(self) -> torch.Tensor:
        """Confidence scores of the last draft block, [B] (proj over [collapsed hidden | markov embed])."""
        B, d = self.cfg.dspark_block_size, self.cfg.dim
        w = self.d_conf[0]
        return self.ws["d_xc"][:B] @ w[:d] + self.ws["d_me_all"] @ w[d:]
