"""One registry of debug switches, parsed once.

The reference reads ~450 environment variables at their use sites, some by presence and some by
value, with defaults that differ per translation unit (``AGENTS.md:49-95``;
``scripts/dsv41_recovery_verify.sh:21-24``).  Here every switch is declared once with a type and a
default, ``FERRITE_<NAME>`` overrides it, and code asks ``switches().name``.
"""
from __future__ import annotations

import os
from dataclasses import dataclass, fields
from typing import Optional


def _parse_bool(v: str) -> bool:
    return v.strip().lower() not in ("", "0", "false", "no", "off")


@dataclass
class Switches:
    timing: bool = False            # per-phase CUDA-event timers in the engines
    layer_sums: bool = False        # per-layer checksums of the residual stream
    trace_tokens: bool = False      # print every emitted token id
    trace_nan: bool = False         # check sublayer outputs for non-finite values (eager runs)
    debug_sync: bool = False        # synchronise after every kernel call
    nvtx: bool = False              # NVTX ranges around engine phases
    pdl: bool = False               # programmatic dependent launch
    ar_group: int = 0               # tiles per published group of the fused GEMV all-reduce (0 = whole grid)
    tc_gemv_min_n: int = 0          # decode GEMVs with at least this many outputs use the tcgen05 split-K kernel (0 = never)
    tc_gemv_max_n: int = 0          # ... and, for 9-16 rows, matrices with at most this many outputs (0 = never)
    # Sublayer-boundary fusions for decode rows, each measured on the GLM decode step (1 GPU / rank 0 of TP=8):
    # fewer launches did not mean a shorter step where the fused stage became a serial tail of its kernel
    fuse_front: bool = False        # next site's hyper-connection front at a grid barrier inside the closing GEMV
                                    # (90 launches fewer, +0.28 / +0.27 ms: the barrier costs more than the launch)
    fuse_route: bool = False        # routing as the tail of the router GEMV
    fuse_swiglu: bool = False       # SwiGLU while the down projection loads its activations (with fuse_route:
                                    # 88 launches fewer, +0.4 / +0.2 ms)
    gdn_own_fg: bool = False        # low-rank decay / gate projections inside the GatedDeltaNet kernel (34 launches
                                    # fewer, +0.04 / +0.12 ms: 8..64 CTAs do serially what a wide GEMV does in parallel)
    hc_pre_wide: bool = True        # hyper-connection front as a column-parallel kernel fed by Gram partials
                                    # (-0.32 / -0.27 ms against the one-CTA-per-row kernel)
    l2_ahead: int = -1              # read-ahead distance of the weight-streaming kernels (-1 = library default)
    gdn_chunk_rows: int = 16        # GatedDeltaNet: groups of at least this many rows use the WY-chunked scan (0 = never)
    moe_tc_rows: int = 64           # GLM routed experts: rows from which the tcgen05 grouped GEMM runs (0 = never)
    d4_mx_min_rows: int = 32        # DSV41 routed experts: rows from which the block-scaled tcgen05 grouped GEMM runs (0 = never);
                                    # 16 rows x 6 experts of 384 are nearly all distinct: grouping them buys no reuse (22.2 vs 16.2 ms per tick)
    d4_tc_min_rows: int = 32        # DSV41 dense projections: rows from which the tcgen05 GEMM replaces 8-row GEMV windows
                                    # (16 rows: two windows, the second from L2, 15.5 vs 16.2 ms per tick)
    d4_fused_rows: int = 8          # DSV41: forwards of up to this many rows close their sublayers with the fused GEMV + all-reduce
                                    # (16: two 8-row windows per launch site, 80 launches fewer per 16-row tick but 15.9 vs 15.5 ms)
    d4_fp4_mma: bool = True         # DSV41 routed experts of decode rows on the tensor cores
    d4_attn_tc: bool = False        # DSV41 tensor-core sparse attention (slower than the SIMT kernel at decode sizes)
    d4_fuse_quant: bool = False     # DSV41 activation quantiser fused into hc_pre (a one-CTA latency chain; slower)
    dump_dir: str = ""              # directory for unit dumps ("" = off)
    allow_stale_kernels: bool = False

    @staticmethod
    def from_env(env=None) -> "Switches":
        env = os.environ if env is None else env
        s = Switches()
        for f in fields(s):
            raw = env.get("FERRITE_" + f.name.upper())
            if raw is None:
                continue
            if f.type in ("bool", bool):
                setattr(s, f.name, _parse_bool(raw))
            elif f.type in ("int", int):
                setattr(s, f.name, int(raw))
            else:
                setattr(s, f.name, raw)
        return s


_CURRENT: Optional[Switches] = None


def switches() -> Switches:
    global _CURRENT
    if _CURRENT is None:
        _CURRENT = Switches.from_env()
    return _CURRENT


def set_switches(s: Optional[Switches]) -> None:
    """Install (or with None: re-read from the environment on next use)."""
    global _CURRENT
    _CURRENT = s
