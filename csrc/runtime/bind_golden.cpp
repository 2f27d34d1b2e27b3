// Python bindings of the f32 CPU golden ops (numpy arrays in, numpy arrays out).
#include <pybind11/numpy.h>
#include <pybind11/pybind11.h>
#include <pybind11/stl.h>

#include "golden.h"
#include "golden_dsv41.h"

namespace py = pybind11;
using farr = py::array_t<float, py::array::c_style | py::array::forcecast>;
using iarr = py::array_t<int64_t, py::array::c_style | py::array::forcecast>;

static farr make(std::vector<py::ssize_t> shape) { return farr(shape); }

void bind_golden(py::module_& m) {
    m.def("matmul", [](farr x, farr w) {
        const int n = (int)x.shape(0), k = (int)x.shape(1), o = (int)w.shape(0);
        farr out = make({n, o});
        golden::matmul(x.data(), w.data(), out.mutable_data(), n, k, o);
        return out;
    });
    m.def("rmsnorm", [](farr x, farr w, float eps) {
        const int n = (int)x.shape(0), d = (int)x.shape(1);
        farr out = make({n, d});
        golden::rmsnorm(x.data(), w.data(), out.mutable_data(), n, d, eps);
        return out;
    });
    m.def("gated_rmsnorm", [](farr o, farr gate, farr w, float eps) {
        const int d = (int)o.shape(o.ndim() - 1);
        const int rows = (int)(o.size() / d);
        farr out(std::vector<py::ssize_t>(o.shape(), o.shape() + o.ndim()));
        golden::gated_rmsnorm(o.data(), gate.data(), w.data(), out.mutable_data(), rows, d, eps);
        return out;
    });
    m.def("swiglu_limited", [](farr gate, farr up, float limit) {
        farr out(std::vector<py::ssize_t>(gate.shape(), gate.shape() + gate.ndim()));
        golden::swiglu_limited(gate.data(), up.data(), out.mutable_data(), (size_t)gate.size(), limit);
        return out;
    });
    m.def("causal_conv1d", [](farr x, farr w, farr state) {
        const int n = (int)x.shape(0), ch = (int)x.shape(1), k = (int)w.shape(1);
        farr out = make({n, ch}), st = make({ch, k - 1});
        golden::causal_conv1d(x.data(), w.data(), state.data(), out.mutable_data(), st.mutable_data(), n, ch, k);
        return py::make_tuple(out, st);
    });
    m.def("gdn_recurrent", [](farr q, farr k, farr v, farr beta, farr g, farr state) {
        const int n = (int)q.shape(0), h = (int)q.shape(1), dk = (int)q.shape(2), dv = (int)v.shape(2);
        farr out = make({n, h, dv});
        farr st = make({h, dk, dv});
        std::copy(state.data(), state.data() + state.size(), st.mutable_data());
        golden::gdn_recurrent(q.data(), k.data(), v.data(), beta.data(), g.data(), st.mutable_data(), out.mutable_data(),
                              n, h, dk, dv);
        return py::make_tuple(out, st);
    });
    m.def("indexer_topk", [](farr q_idx, farr keys, farr w, int topk, int ctx0) {
        const int n = (int)q_idx.shape(0), H = (int)q_idx.shape(1), D = (int)q_idx.shape(2), t = (int)keys.shape(0);
        iarr idx({(py::ssize_t)n, (py::ssize_t)topk});
        golden::indexer_topk(q_idx.data(), keys.data(), w.data(), n, H, D, t, topk, ctx0, idx.mutable_data());
        return idx;
    });
    m.def("sparse_mla_attn", [](farr q, farr k, farr v, iarr idx, bool with_lse) -> py::object {
        const int n = (int)q.shape(0), h = (int)q.shape(1), d = (int)q.shape(2), t = (int)k.shape(0), dv = (int)v.shape(2);
        const int W = (int)idx.shape(1);
        farr out = make({n, h, dv}), lse = make({n, h});
        golden::sparse_mla_attn(q.data(), k.data(), v.data(), idx.data(), out.mutable_data(),
                                with_lse ? lse.mutable_data() : nullptr, n, h, d, dv, t, W);
        if (with_lse) return py::make_tuple(out, lse);
        return std::move(out);
    }, py::arg("q"), py::arg("k"), py::arg("v"), py::arg("idx"), py::arg("with_lse") = false);
    m.def("lse_merge", [](farr outs, farr lses) {
        const int S = (int)outs.shape(0), dv = (int)outs.shape(outs.ndim() - 1);
        const int rows = (int)(outs.size() / S / dv);
        std::vector<py::ssize_t> shp(outs.shape() + 1, outs.shape() + outs.ndim());
        farr merged(shp);
        golden::lse_merge(outs.data(), lses.data(), merged.mutable_data(), S, rows, dv);
        return merged;
    });
    m.def("moe_route", [](farr logits, farr bias, int topk, float scaling) {
        const int n = (int)logits.shape(0), E = (int)logits.shape(1);
        farr wts = make({n, topk});
        iarr ids({(py::ssize_t)n, (py::ssize_t)topk});
        golden::moe_route(logits.data(), bias.data(), n, E, topk, scaling, wts.mutable_data(), ids.mutable_data());
        return py::make_tuple(wts, ids);
    });
    m.def("hc_pre", [](farr R, farr fn, farr scale, farr base, float rms_eps, float hc_eps, int iters) {
        const int T = (int)R.shape(0), n = (int)R.shape(1), H = (int)R.shape(2);
        farr x = make({T, H}), post = make({T, n}), comb = make({T, n, n});
        golden::hc_pre(R.data(), fn.data(), scale.data(), base.data(), x.mutable_data(), post.mutable_data(),
                       comb.mutable_data(), T, n, H, rms_eps, hc_eps, iters);
        return py::make_tuple(x, post, comb);
    });
    m.def("hc_post", [](farr y, farr R, farr post, farr comb) {
        const int T = (int)R.shape(0), n = (int)R.shape(1), H = (int)R.shape(2);
        farr out = make({T, n, H});
        golden::hc_post(y.data(), R.data(), post.data(), comb.data(), out.mutable_data(), T, n, H);
        return out;
    });
    m.def("argmax_first", [](farr x) { return golden::argmax_first(x.data(), (int)x.size()); });
    m.def("spec_accept", [](std::vector<int64_t> drafts, std::vector<int64_t> judges, bool anchor_in_block) {
        return golden::spec_accept(drafts.data(), (int)drafts.size(), judges.data(), (int)judges.size(), anchor_in_block);
    });
    // ---- DSV41 family ----------------------------------------------------------------------------
    m.def("d4_e4m3_round", [](farr x) {
        farr out(std::vector<py::ssize_t>(x.shape(), x.shape() + x.ndim()));
        for (py::ssize_t i = 0; i < x.size(); ++i) out.mutable_data()[i] = golden_d4::e4m3_round(x.data()[i]);
        return out;
    });
    m.def("d4_e2m1_round", [](farr x) {
        farr out(std::vector<py::ssize_t>(x.shape(), x.shape() + x.ndim()));
        for (py::ssize_t i = 0; i < x.size(); ++i) out.mutable_data()[i] = golden_d4::e2m1_round(x.data()[i]);
        return out;
    });
    m.def("d4_fp8_act_roundtrip", [](farr x, int block) {
        farr out(std::vector<py::ssize_t>(x.shape(), x.shape() + x.ndim()));
        std::copy(x.data(), x.data() + x.size(), out.mutable_data());
        golden_d4::fp8_act_roundtrip(out.mutable_data(), (size_t)x.size(), block);
        return out;
    });
    m.def("d4_fp4_act_roundtrip", [](farr x, int block, bool e4m3_scale) {
        farr out(std::vector<py::ssize_t>(x.shape(), x.shape() + x.ndim()));
        std::copy(x.data(), x.data() + x.size(), out.mutable_data());
        golden_d4::fp4_act_roundtrip(out.mutable_data(), (size_t)x.size(), block, e4m3_scale);
        return out;
    });
    m.def("d4_sparse_attn_sink", [](farr q, farr kv, farr sink, float scale) {
        const int H = (int)q.shape(0), d = (int)q.shape(1), n = (int)kv.shape(0);
        farr out = make({H, d});
        golden_d4::sparse_attn_sink(q.data(), kv.data(), sink.data(), out.mutable_data(), H, d, n, scale);
        return out;
    });
    m.def("d4_route", [](farr logits, farr bias, int topk, float route_scale) {
        const int n = (int)logits.shape(0), E = (int)logits.shape(1);
        iarr idx({(py::ssize_t)n, (py::ssize_t)topk});
        farr wts = make({n, topk});
        golden_d4::route_sqrtsoftplus(logits.data(), bias.data(), n, E, topk, route_scale, idx.mutable_data(), wts.mutable_data());
        return py::make_tuple(wts, idx);
    });
    m.def("d4_candidate_blocks", [](farr score, int clen, int topk_blocks, int bs) {
        const int n = (int)score.shape(0);
        py::array_t<uint8_t> keep({(py::ssize_t)n});
        golden_d4::candidate_blocks(score.data(), n, clen, topk_blocks, bs, keep.mutable_data());
        return keep;
    });
}
