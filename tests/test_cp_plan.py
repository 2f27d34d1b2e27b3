"""CPU: layout math of the context-parallel prefill group and its hand-off (no device work)."""
import pytest

from ferrite_b200.config import GlmConfig
from ferrite_b200.parallel.cp import cp_layer_range, stage_parts
from ferrite_b200.parallel.pdaf import TransferPlan


@pytest.mark.parametrize("n_layers,n_stages", [(45, 4), (45, 8), (4, 2), (7, 7), (10, 3)])
def test_layer_ranges_are_contiguous_balanced_and_complete(n_layers, n_stages):
    ranges = [cp_layer_range(n_layers, n_stages, s) for s in range(n_stages)]
    assert ranges[0][0] == 0 and ranges[-1][1] == n_layers
    assert all(a[1] == b[0] for a, b in zip(ranges, ranges[1:]))
    sizes = [b - a for a, b in ranges]
    assert max(sizes) - min(sizes) <= 1 and sizes == sorted(sizes, reverse=True)


def test_every_cache_family_and_state_has_exactly_one_owner_stage():
    cfg = GlmConfig.production()
    for n_stages in (1, 2, 4):
        fams, gidx = [], []
        for s in range(n_stages):
            f, g = stage_parts(cfg, *cp_layer_range(cfg.num_layers, n_stages, s))
            fams += f
            gidx += g
        assert sorted(gidx) == list(range(len(cfg.linear_layers)))          # every recurrent state travels once
        assert sorted(set(fams)) == list(range(cfg.n_dsa_families))          # every paged family is exported
        # the MTP layer's family goes with the last stage
        last_f, _ = stage_parts(cfg, *cp_layer_range(cfg.num_layers, n_stages, n_stages - 1))
        assert cfg.dsa_family(cfg.num_layers) in last_f


@pytest.mark.parametrize("n_tokens,ps,n_dcp", [(45, 16, 2), (4096, 64, 4), (1, 16, 4), (65536, 64, 4)])
def test_dcp_page_split_is_a_partition_with_compact_slots(n_tokens, ps, n_dcp):
    plans = [TransferPlan(n_tokens, ps, n_dcp, d) for d in range(n_dcp)]
    pages = sorted(p for pl in plans for p in pl.src_pages)
    assert pages == list(range(plans[0].n_pages))                             # every page to exactly one rank
    for pl in plans:
        assert pl.dst_slots == list(range(len(pl.src_pages)))                 # compact: no holes on the decode rank
        assert all(p % n_dcp == pl.d for p in pl.src_pages)
    per = [len(pl.src_pages) for pl in plans]
    assert max(per) - min(per) <= 1
