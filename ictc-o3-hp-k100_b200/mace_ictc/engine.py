"""Force engine: energy and position gradient of the MACE-ICTC model by an explicit forward and reverse
sweep over the B200 kernels, without the autograd tape.

Same arithmetic as ``MaceIctcModel.forward`` followed by ``autograd.grad(E, pos)``
(reference: mace_ictc/hp/runtime.py:82-111 over mace_ictc/models/mace/backbone.py:860-1246), specialised to
what an MD step needs: frozen weights, gradient with respect to positions only.  Every adjoint below is
the hand-written reverse of the line that produced the value; tests compare it with the autograd path.
Node features live in ir_mul rows ([rows, 9C], degree blocks [2l+1, C]) from end to end, so channel
linears are plain GEMMs over contiguous rows and no mul_ir <-> ir_mul conversion is made.
Dense layers are fp32 library GEMMs (``torch.mm``).
"""
from __future__ import annotations

import ctypes as C
import math

import torch

from ictc_o3 import _lib
from ictc_o3.ops.topology import build_csr
from ictc_o3.symmetric_contraction import _ScCall
from . import domain as D
from .model import SILU_SCALE, MaceIctcModel


def _blocks(flat, c):
    """Views of the three degree blocks of ir_mul rows [rows, 9C] as [rows, m, C]."""
    rows = flat.shape[0]
    return [flat[:, 0:c].reshape(rows, 1, c), flat[:, c:4 * c].reshape(rows, 3, c),
            flat[:, 4 * c:9 * c].reshape(rows, 5, c)]


class ForceEngine:
    def __init__(self, model: MaceIctcModel):
        if len(model.interactions) != 2:
            raise ValueError("the force engine covers the two-interaction model")
        self.model = model
        self.c = model.channels
        self.dev = next(model.parameters()).device
        self.lib = _lib.load()
        self._versions = None
        self._spec = {0: _lib.tp_spec(0, 2, 2), 1: _lib.tp_spec(2, 2, 2)}
        self.fused_mlp = True
        self.gate_gemm = True    # last MLP layer on the tcgen05 tensor cores (False: single mma.sync kernel)
        self.mlp_chain = True    # hidden MLP layers as a TMEM chain (False: mma.sync kernels)
        self.tc_linear = True    # per-degree channel linears on the same kernels (False: library fp32 GEMM)
        self.profile = None      # list of (kernel name, start event, end event) when enabled by a benchmark
        self.refresh()

    # ---------------------------------------------------------------- weights
    def refresh(self):
        """(Re)build the GEMM-ready weight views when a parameter changed."""
        versions = tuple(p._version for p in self.model.parameters())
        if versions == self._versions:
            return
        m, c = self.model, self.c
        with torch.no_grad():
            self.emb = m.node_embedding.weight.t().contiguous()                         # [S, C]
            self.layers = []
            for k, (inter, prod) in enumerate(zip(m.interactions, m.products)):
                lin = inter.input_lmax
                L = {
                    "up_t": [inter.linear_up.adapters[str(l)].weight.t().contiguous() for l in range(lin + 1)],
                    "up": [inter.linear_up.adapters[str(l)].weight.contiguous() for l in range(lin + 1)],
                    "fc": [mod.weight.contiguous() for mod in inter.fc if isinstance(mod, torch.nn.Linear)],
                    "fc_t": [mod.weight.t().contiguous() for mod in inter.fc if isinstance(mod, torch.nn.Linear)],
                    "ml": [(inter.message_linear.weights[str(l)] / max(inter.avg_num_neighbors, 1e-8)).contiguous()
                           for l in range(3)],
                    "counts": [inter.tp.path_counts_by_l[l] for l in range(3)],
                    "tpw": None if bool(torch.all(inter.tp.weight == 1)) else inter.tp.weight.contiguous(),
                }
                L["ml_t"] = [w.t().contiguous() for w in L["ml"]]
                L["w3_split"] = self._split(L["fc"][-1])
                L["w3t_split"] = self._split(L["fc_t"][-1])
                if self._fused_mlp_ok(L) and self.gate_gemm:
                    L["w3_umma"] = self._pack_umma(L["fc"][-1], 0)
                    L["w3t_umma"] = self._pack_umma(L["fc"][-1], 1)
                    L["hid_umma"] = [self._pack_umma(L["fc"][1], 0), self._pack_umma(L["fc"][2], 0)]
                    L["hid_t_umma"] = [self._pack_umma(L["fc"][1], 1), self._pack_umma(L["fc"][2], 1)]
                wsc = inter.self_connection.weights["0"]                                 # [S, C(out), C(in)]
                s = wsc.shape[0]
                L["sc_fwd"] = wsc.permute(2, 0, 1).reshape(c, s * c).contiguous()          # x @ -> [n, S*C(out)]
                L["sc_bwd"] = wsc.permute(1, 0, 2).reshape(c, s * c).contiguous()          # dout @ -> [n, S*C(in)]
                L["bank"] = prod.symmetric_contractions.weight_bank()
                L["target"] = prod.target_lmax
                L["pl"] = [(prod.linear[str(l)] / math.sqrt(c)).contiguous() for l in range(prod.target_lmax + 1)]
                L["pl_t"] = [w.t().contiguous() for w in L["pl"]]
                if self.tc_linear and c == 64:
                    # operand-layout copies for the tensor-core channel linears: key -> (packed, k_chunks, n_chunks)
                    P = {}
                    for l in range(lin + 1):
                        P["up", l] = self._pack_lin(L["up"][l], L["up_t"][l])
                        P["up_b", l] = self._pack_lin(L["up_t"][l], L["up"][l])
                    for l in range(3):
                        P["ml", l] = self._pack_lin(L["ml"][l], L["ml_t"][l])        # x @ ml_t
                        P["ml_b", l] = self._pack_lin(L["ml_t"][l], L["ml"][l])      # x @ ml
                    for l in range(prod.target_lmax + 1):
                        P["pl", l] = self._pack_lin(L["pl_t"][l], L["pl"][l])        # x @ pl
                        P["pl_b", l] = self._pack_lin(L["pl"][l], L["pl_t"][l])      # x @ pl_t
                    L["packed"] = P
                self.layers.append(L)
            self.ro0 = m.layer_energy_readouts[0].readout.weight.reshape(-1).contiguous()  # [C]
            self.ro1_w1 = m.last_layer_energy_readout.linear_1.weight.contiguous()          # [16, C]
            self.ro1_w2 = m.last_layer_energy_readout.linear_2.weight.reshape(-1).contiguous()  # [16]
        self._versions = versions

    def _split(self, w):
        """{tf32(x), tf32(x - tf32(x))} pairs of a weight matrix for the tensor-core MLP kernels."""
        out = torch.empty(*w.shape, 2, dtype=torch.float32, device=w.device)
        with _lib.on_device(w.device):
            _lib.check(self.lib.ictc_split_tf32(w.numel(), w.data_ptr(), out.data_ptr(), _lib.stream(w.device)),
                       "split_tf32")
        return out

    def _pack_umma(self, w, transpose):
        """Last-layer weights in the shared-memory operand layout of the tcgen05 gate GEMM kernels."""
        out = torch.empty(2 * w.numel(), dtype=torch.float32, device=w.device)
        with _lib.on_device(w.device):
            _lib.check(self.lib.ictc_gate_pack_weights(w.shape[0], w.data_ptr(), transpose, out.data_ptr(),
                                                       _lib.stream(w.device)), "gate_pack_weights")
        return out

    def _pack_lin(self, w_out_major, w_in_major):
        """Operand copy for out = x @ w_in_major, where w_in_major is [K, N] and w_out_major its transpose."""
        k, n = w_in_major.shape
        if k == 64:
            return self._pack_umma(w_out_major.contiguous(), 0), 1, n // 64
        if n != 64:
            raise ValueError("tensor-core channel linear needs a 64-wide side")
        return self._pack_umma(w_in_major.contiguous(), 1), k // 64, 1

    def _lin(self, L, key, rows, in_t, in_off, in_mm, in_ld, out_t, out_off, out_mm, out_ld):
        """out rows = in rows @ W on the tensor cores, reading / writing per-degree blocks in place."""
        packed, kc, nc = L["packed"][key]
        t0 = self._mark()
        _lib.check(self.lib.ictc_channel_linear_tc(rows, kc, nc, in_t.data_ptr() + 4 * in_off, in_mm, in_ld,
                                                   packed.data_ptr(), out_t.data_ptr() + 4 * out_off, out_mm, out_ld,
                                                   self._st()), "channel_linear_tc")
        self._done("channel_linear_tc", t0)

    # ---------------------------------------------------------------- buffers
    @staticmethod
    def bucket(rows):
        """Row count rounded up to 1/16 of its power of two.  Edge and atom counts change a little every MD step;
        allocating the rounded size keeps the sizes repeating, so the caching allocator reuses its blocks
        instead of splitting, freeing and re-allocating multi-GB segments."""
        rows = int(rows)
        if rows <= 4096:
            return 4096
        g = 1 << (rows.bit_length() - 5)
        return (rows + g - 1) // g * g

    def _rows(self, rows, *cols, zero=False):
        make = torch.zeros if zero else torch.empty
        return make(self.bucket(rows), *cols, dtype=torch.float32, device=self.dev)[:rows]

    # ---------------------------------------------------------------- small launch helpers
    def _st(self):
        return _lib.stream(self.dev)

    def _silu(self, x):
        y = torch.empty_like(x)
        _lib.check(self.lib.ictc_silu_forward(x.numel(), SILU_SCALE, x.data_ptr(), y.data_ptr(), self._st()), "silu")
        return y

    def _silu_bwd(self, x, dy):
        dx = torch.empty_like(x)
        _lib.check(self.lib.ictc_silu_backward(x.numel(), SILU_SCALE, x.data_ptr(), dy.data_ptr(), dx.data_ptr(),
                                               self._st()), "silu_backward")
        return dx

    def _fused_mlp_ok(self, L):
        fc = L["fc"]
        return (self.fused_mlp and len(fc) == 4 and fc[0].shape[0] == 64 and fc[0].shape[1] <= 8
                and tuple(fc[1].shape) == (64, 64) and tuple(fc[2].shape) == (64, 64)
                and fc[3].shape[1] == 64 and fc[3].shape[0] % 64 == 0)

    def _chain_ok(self, L):
        return self._fused_mlp_ok(L) and "w3_umma" in L and self.mlp_chain

    def _mlp(self, rb, L, rows=None, limit=None):
        """Radial MLP: returns gates and the pre-activations needed by the reverse sweep.  ``rows`` (tensor-memory
        chain kernels only) makes row r of the MLP read rb[rows[r]]; ``limit`` is a device scalar with the number
        of rows that are really in use (fixed-capacity buffers of a recorded step)."""
        if self._fused_mlp_ok(L):
            e, fc = (rb.shape[0] if rows is None else rows.numel()), L["fc"]
            nout = fc[3].shape[0]
            gates = self._rows(e, nout)
            pre = [self._rows(e, 64) for _ in range(3)]
            t0 = self._mark()
            if "w3_umma" in L:
                if self.mlp_chain:
                    _lib.check(self.lib.ictc_mlp_chain_forward(e, rb.shape[1], _lib.ptr(rb), _lib.ptr(rows),
                                                               fc[0].data_ptr(),
                                                               L["hid_umma"][0].data_ptr(), L["hid_umma"][1].data_ptr(),
                                                               _lib.ptr(pre[0]), _lib.ptr(pre[1]), _lib.ptr(pre[2]),
                                                               _lib.ptr(limit), self._st()), "mlp_chain_forward")
                else:
                    _lib.check(self.lib.ictc_radial_mlp_hidden_forward(e, rb.shape[1], _lib.ptr(rb), fc[0].data_ptr(),
                                                                       fc[1].data_ptr(), fc[2].data_ptr(),
                                                                       _lib.ptr(pre[0]), _lib.ptr(pre[1]),
                                                                       _lib.ptr(pre[2]), self._st()),
                               "radial_mlp_hidden_forward")
                self._done(f"radial_mlp_hidden_forward_{nout}", t0)
                t0 = self._mark()
                _lib.check(self.lib.ictc_gate_gemm_forward(e, nout, _lib.ptr(pre[2]), L["w3_umma"].data_ptr(),
                                                           _lib.ptr(gates), 1, _lib.ptr(limit), self._st()),
                           "gate_gemm_forward")
                self._done(f"gate_gemm_forward_{nout}", t0)
                return gates, pre
            _lib.check(self.lib.ictc_radial_mlp_forward(e, rb.shape[1], nout, _lib.ptr(rb), fc[0].data_ptr(),
                                                        fc[1].data_ptr(), fc[2].data_ptr(), L["w3_split"].data_ptr(),
                                                        _lib.ptr(gates), _lib.ptr(pre[0]), _lib.ptr(pre[1]),
                                                        _lib.ptr(pre[2]), self._st()), "radial_mlp_forward")
            self._done(f"radial_mlp_forward_{nout}", t0)
            return gates, pre
        pre, h = [], rb
        for k, wt in enumerate(L["fc_t"]):
            z = torch.mm(h, wt)
            if k + 1 < len(L["fc_t"]):
                pre.append(z)
                h = self._silu(z)
            else:
                return z, pre

    def _mlp_bwd(self, dgates, pre, L, pairs=None, out=None, accumulate=False, limit=None):
        """Input gradient of the radial MLP.  With ``out`` [E, num_basis] (chain kernels, paired rows) the result of
        pair u is written or added to out[rep_edge[u]] and ``out`` is returned."""
        if pairs is not None and not self._fused_mlp_ok(L):
            dgates = dgates.index_select(0, pairs[1]) + torch.where(
                (pairs[2] >= 0).unsqueeze(1), dgates.index_select(0, pairs[2].clamp_min(0)), dgates.new_zeros(()))
            pairs = None
        if self._fused_mlp_ok(L):
            ft = L["fc_t"]
            e = pre[0].shape[0]
            nb = ft[0].shape[0]
            drb = self._rows(e, nb) if out is None else out
            t0 = self._mark()
            pa, pb = (None, None) if pairs is None else (pairs[1], pairs[2])
            if "w3t_umma" in L:
                da3 = self._rows(e, 64)
                _lib.check(self.lib.ictc_gate_gemm_backward(e, dgates.shape[1], _lib.ptr(dgates), _lib.ptr(pa),
                                                            _lib.ptr(pb), L["w3t_umma"].data_ptr(), _lib.ptr(da3),
                                                            _lib.ptr(limit), self._st()), "gate_gemm_backward")
                self._done(f"gate_gemm_backward_{dgates.shape[1]}", t0)
                t0 = self._mark()
                if self.mlp_chain:
                    _lib.check(self.lib.ictc_mlp_chain_backward(e, nb, _lib.ptr(da3), L["fc"][0].data_ptr(),
                                                                L["hid_t_umma"][0].data_ptr(),
                                                                L["hid_t_umma"][1].data_ptr(), _lib.ptr(pre[0]),
                                                                _lib.ptr(pre[1]), _lib.ptr(pre[2]), _lib.ptr(drb),
                                                                _lib.ptr(pa) if out is not None else None,
                                                                int(accumulate), _lib.ptr(limit), self._st()),
                               "mlp_chain_backward")
                else:
                    _lib.check(self.lib.ictc_radial_mlp_hidden_backward(e, nb, _lib.ptr(da3), ft[0].data_ptr(),
                                                                        ft[1].data_ptr(), ft[2].data_ptr(),
                                                                        _lib.ptr(pre[0]), _lib.ptr(pre[1]),
                                                                        _lib.ptr(pre[2]), _lib.ptr(drb), self._st()),
                               "radial_mlp_hidden_backward")
                self._done(f"radial_mlp_hidden_backward_{dgates.shape[1]}", t0)
                return drb
            _lib.check(self.lib.ictc_radial_mlp_backward_paired(e, nb, dgates.shape[1], _lib.ptr(dgates), _lib.ptr(pa),
                                                                _lib.ptr(pb), ft[0].data_ptr(),
                                                                ft[1].data_ptr(), ft[2].data_ptr(),
                                                                L["w3t_split"].data_ptr(), _lib.ptr(pre[0]),
                                                                _lib.ptr(pre[1]), _lib.ptr(pre[2]), _lib.ptr(drb),
                                                                self._st()), "radial_mlp_backward")
            self._done(f"radial_mlp_backward_{dgates.shape[1]}", t0)
            return drb
        d = torch.mm(dgates, L["fc"][-1])
        for k in range(len(pre) - 1, -1, -1):
            d = self._silu_bwd(pre[k], d)
            d = torch.mm(d, L["fc"][k])
        return d                                                            # [E, num_basis]

    def _species_linear(self, x, species, w, s):
        full = torch.mm(x, w).view(x.shape[0], s, self.c)
        return full.gather(1, species.view(-1, 1, 1).expand(-1, 1, self.c)).squeeze(1)

    def _mark(self):
        if self.profile is None:
            return None
        ev = torch.cuda.Event(enable_timing=True)
        ev.record(torch.cuda.current_stream(self.dev))
        return ev

    def _done(self, name, start):
        if start is not None:
            self.profile.append((name, start, self._mark()))

    def _tp_forward(self, layer, x, sh, g, src, rowptr, rows, e, tpw, grow=None):
        c = self.c
        out = self._rows(rows, (9 if layer == 0 else 35) * c)
        t0 = self._mark()
        _lib.check(self.lib.ictc_tp_graph_forward_shared(self._spec[layer], c, rows, e, x.data_ptr(), sh.data_ptr(),
                                                         _lib.ptr(tpw), g.data_ptr(), _lib.ptr(grow), src.data_ptr(),
                                                         rowptr.data_ptr(), None, None, out.data_ptr(), self._st()),
                   "tp_graph_forward")
        self._done(f"graph_forward_l{layer}", t0)
        return out

    def _tp_adjoint(self, layer, x, sh, g, dst, src_csr, v, n_rows, e, tpw, need_x, grow=None):
        c = self.c
        dx = self._rows(x.shape[0], x.shape[1]) if need_x else None
        dsh = self._rows(e, 9)
        dg = self._rows(e, g.shape[1])
        rowptr, order = src_csr
        t0 = self._mark()
        _lib.check(self.lib.ictc_tp_graph_adjoint_shared(self._spec[layer], c, n_rows, e, x.data_ptr(), sh.data_ptr(),
                                                         _lib.ptr(tpw), g.data_ptr(), _lib.ptr(grow), dst.data_ptr(),
                                                         rowptr.data_ptr(), _lib.ptr(order), None, v.data_ptr(),
                                                         _lib.ptr(dx), dsh.data_ptr(), dg.data_ptr(), self._st()),
                   "tp_graph_adjoint")
        self._done(f"graph_adjoint_l{layer}", t0)
        return dx, dsh, dg

    def _transpose(self, rows, count, m, in_t, in_off, in_stride, out_t, out_off, out_stride, to_gemm):
        _lib.check(self.lib.ictc_slot_transpose(rows, count, m, self.c, in_stride, out_stride,
                                                in_t.data_ptr() + 4 * in_off, out_t.data_ptr() + 4 * out_off,
                                                int(to_gemm), self._st()), "slot_transpose")

    # ---------------------------------------------------------------- the sweep
    @torch.no_grad()
    def energy_and_gradient(self, pos, species, src, dst, shifts, box, n_owned, dst_rowptr, plan=None, n_rows=None,
                            pairs=None):
        """pos [N_local,3] (owned rows first), species [N_local] (index), edges sorted by receiver with all
        receivers < n_owned, dst_rowptr [n_owned+1].  Returns (energy of owned atoms, dE/dpos [N_local,3],
        per-atom energies [n_owned]).  ``n_rows`` < N_local marks trailing rows of ``pos`` as padding: they may
        be named by inert edges (whose sender index is then outside the sender CSR) but carry no features.
        ``pairs`` = (gate_row [E], rep_edge [U], other_edge [U]) evaluates the radial MLP once per edge pair; an
        optional fourth element is a device int64 scalar with the number of pair rows in use when U is a capacity."""
        self.refresh()
        m, c, lib, dev = self.model, self.c, self.lib, self.dev
        n_local, e = (pos.shape[0] if n_rows is None else int(n_rows)), int(src.numel())
        species = species[:n_local]
        st = self._st()
        L0, L1 = self.layers
        nb, pcut, rmax = m.number_of_basis, m.polynomial_cutoff_p, m.max_radius
        with _lib.on_device(dev):
            # ---- edge geometry
            sh = self._rows(e, 9)
            rb = self._rows(e, nb)
            unit = self._rows(e, 3)
            length = self._rows(e)
            box_c = (C.c_float * 3)(*[float(b) for b in box])
            _lib.check(lib.ictc_edge_geometry_forward(pos.data_ptr(), _lib.ptr(src), _lib.ptr(dst), _lib.ptr(shifts),
                                                      box_c, rmax, nb, pcut, e, _lib.ptr(sh), _lib.ptr(rb),
                                                      _lib.ptr(unit), _lib.ptr(length), st), "edge_geometry_forward")
            src_csr = build_csr(src, n_local, assume_sorted=False)
            grow = None if pairs is None else pairs[0]
            by_rows = pairs is not None and self._chain_ok(L0) and self._chain_ok(L1)
            rb_rows = pairs[1] if by_rows else None          # the MLP kernels gather / scatter the pair rows
            live = pairs[3] if (by_rows and len(pairs) > 3) else None   # device count of pair rows in use
            rb_u = rb if (pairs is None or by_rows) else rb.index_select(0, pairs[1])
            sp_owned = species[:n_owned]
            s_count = self.emb.shape[0]
            # ---- layer 0
            x0 = self.emb.index_select(0, species)                               # [N_local, C]
            tc = "packed" in L0 and "packed" in L1
            if tc:
                u0 = self._rows(n_local, c)
                self._lin(L0, ("up", 0), n_local, x0, 0, 1, c, u0, 0, 1, c)
            else:
                u0 = torch.mm(x0, L0["up_t"][0])
            g0, pre0 = self._mlp(rb_u, L0, rb_rows, live)
            M0 = self._tp_forward(0, u0, sh, g0, src, dst_rowptr, n_owned, e, L0["tpw"], grow)   # [n, 9C]
            m0 = self._rows(n_owned, 9 * c)
            for l, (off, mm) in enumerate(((0, 1), (1, 3), (4, 5))):
                if tc:
                    self._lin(L0, ("ml", l), n_owned * mm, M0, off * c, mm, 9 * c, m0, off * c, mm, 9 * c)
                    continue
                m0[:, off * c:(off + mm) * c] = torch.mm(M0[:, off * c:(off + mm) * c].reshape(-1, c),
                                                         L0["ml_t"][l]).view(n_owned, mm * c)
            sc0 = self._species_linear(x0[:n_owned], sp_owned, L0["sc_fwd"], s_count)
            call0 = _ScCall(c, 2, s_count, sp_owned, True)
            y0 = call0.forward(m0, L0["bank"])                                    # [n, 9C]
            h1 = self._rows(n_owned, 9 * c)
            for l, (off, mm) in enumerate(((0, 1), (1, 3), (4, 5))):
                if tc:
                    self._lin(L0, ("pl", l), n_owned * mm, y0, off * c, mm, 9 * c, h1, off * c, mm, 9 * c)
                    continue
                h1[:, off * c:(off + mm) * c] = torch.mm(y0[:, off * c:(off + mm) * c].reshape(-1, c),
                                                         L0["pl"][l]).view(n_owned, mm * c)
            h1[:, :c] += sc0
            e0 = torch.mv(h1[:, :c], self.ro0)
            # ---- halo: the ghost rows travel while the layer-1 gates (which need only the radial basis) are computed
            halo = None if plan is None else plan.forward_async(h1)
            g1, pre1 = self._mlp(rb_u, L1, rb_rows, live)
            h1_full = h1 if plan is None else torch.cat((h1, halo()), 0)
            # ---- layer 1
            u1 = self._rows(n_local, 9 * c)
            for l, (off, mm) in enumerate(((0, 1), (1, 3), (4, 5))):
                if tc:
                    self._lin(L1, ("up", l), n_local * mm, h1_full, off * c, mm, 9 * c, u1, off * c, mm, 9 * c)
                    continue
                u1[:, off * c:(off + mm) * c] = torch.mm(h1_full[:, off * c:(off + mm) * c].reshape(-1, c),
                                                         L1["up_t"][l]).view(n_local, mm * c)
            M1 = self._tp_forward(1, u1, sh, g1, src, dst_rowptr, n_owned, e, L1["tpw"], grow)   # [n, 35C]
            m1 = self._rows(n_owned, 9 * c)
            in_off = 0
            for l, (off, mm) in enumerate(((0, 1), (1, 3), (4, 5))):
                cnt = L1["counts"][l]
                if tc:      # the slot-major block is contracted in place: no transposed copy
                    self._lin(L1, ("ml", l), n_owned * mm, M1, in_off, mm, 35 * c, m1, off * c, mm, 9 * c)
                else:
                    buf = torch.empty(n_owned * mm, cnt * c, dtype=torch.float32, device=dev)
                    self._transpose(n_owned, cnt, mm, M1, in_off, 35 * c, buf, 0, mm * cnt * c, True)
                    m1[:, off * c:(off + mm) * c] = torch.mm(buf, L1["ml_t"][l]).view(n_owned, mm * c)
                in_off += cnt * mm * c
            sc1 = self._species_linear(h1[:, :c].contiguous(), sp_owned, L1["sc_fwd"], s_count)
            call1 = _ScCall(c, 0, s_count, sp_owned, True)
            y1 = call1.forward(m1, L1["bank"])                                    # [n, C]
            h2 = torch.mm(y1, L1["pl"][0]) + sc1
            z = torch.mm(h2, self.ro1_w1.t())
            a = self._silu(z)
            e1 = torch.mv(a, self.ro1_w2)
            atomic = e0 + e1
            energy = atomic.sum()

            # ================= reverse sweep (dE = 1 for every owned atom) =================
            da = self.ro1_w2.unsqueeze(0).expand(n_owned, -1).contiguous()
            dz = self._silu_bwd(z, da)
            dh2 = torch.mm(dz, self.ro1_w1)                                        # [n, C]
            dy1 = torch.mm(dh2, L1["pl_t"][0])
            dm1, _ = call1.adjoint(m1, L1["bank"], dy1, (True, False))             # [n, 9C]
            v1 = self._rows(n_owned, 35 * c)
            out_off = 0
            for l, (off, mm) in enumerate(((0, 1), (1, 3), (4, 5))):
                cnt = L1["counts"][l]
                if tc:
                    self._lin(L1, ("ml_b", l), n_owned * mm, dm1, off * c, mm, 9 * c, v1, out_off, mm, 35 * c)
                else:
                    buf = torch.mm(dm1[:, off * c:(off + mm) * c].reshape(-1, c), L1["ml"][l])   # [n*mm, cnt*C]
                    self._transpose(n_owned, cnt, mm, buf, 0, mm * cnt * c, v1, out_off, 35 * c, False)
                out_off += cnt * mm * c
            du1, dsh1, dg1 = self._tp_adjoint(1, u1, sh, g1, dst, src_csr, v1, n_local, e, L1["tpw"], True, grow)
            dh1_full = self._rows(n_local, 9 * c)
            for l, (off, mm) in enumerate(((0, 1), (1, 3), (4, 5))):
                if tc:
                    self._lin(L1, ("up_b", l), n_local * mm, du1, off * c, mm, 9 * c, dh1_full, off * c, mm, 9 * c)
                    continue
                dh1_full[:, off * c:(off + mm) * c] = torch.mm(du1[:, off * c:(off + mm) * c].reshape(-1, c),
                                                               L1["up"][l]).view(n_local, mm * c)
            # the ghost rows' cotangents travel back while the layer-1 MLP is differentiated
            halo = None if plan is None else plan.adjoint_async(dh1_full[n_owned:].contiguous())
            drb = self._rows(e, nb, zero=True) if by_rows else None
            drb = self._mlp_bwd(dg1, pre1, L1, pairs, drb, False, live)
            del dg1, g1, pre1
            dh1 = dh1_full[:n_owned]
            if plan is not None:
                dh1 = dh1 + halo()
            else:
                dh1 = dh1.clone()
            dsc1 = dh2
            full = torch.mm(dsc1, L1["sc_bwd"]).view(n_owned, s_count, c)
            dh1[:, :c] += full.gather(1, sp_owned.view(-1, 1, 1).expand(-1, 1, c)).squeeze(1)
            dh1[:, :c] += self.ro0
            dy0 = self._rows(n_owned, 9 * c)
            for l, (off, mm) in enumerate(((0, 1), (1, 3), (4, 5))):
                if tc:
                    self._lin(L0, ("pl_b", l), n_owned * mm, dh1, off * c, mm, 9 * c, dy0, off * c, mm, 9 * c)
                    continue
                dy0[:, off * c:(off + mm) * c] = torch.mm(dh1[:, off * c:(off + mm) * c].reshape(-1, c),
                                                          L0["pl_t"][l]).view(n_owned, mm * c)
            dm0, _ = call0.adjoint(m0, L0["bank"], dy0, (True, False))
            v0 = self._rows(n_owned, 9 * c)
            for l, (off, mm) in enumerate(((0, 1), (1, 3), (4, 5))):
                if tc:
                    self._lin(L0, ("ml_b", l), n_owned * mm, dm0, off * c, mm, 9 * c, v0, off * c, mm, 9 * c)
                    continue
                v0[:, off * c:(off + mm) * c] = torch.mm(dm0[:, off * c:(off + mm) * c].reshape(-1, c),
                                                         L0["ml"][l]).view(n_owned, mm * c)
            _, dsh0, dg0 = self._tp_adjoint(0, u0, sh, g0, dst, src_csr, v0, n_local, e, L0["tpw"], False, grow)
            if by_rows:
                self._mlp_bwd(dg0, pre0, L0, pairs, drb, True, live)
            else:
                drb += self._mlp_bwd(dg0, pre0, L0, pairs)
                if pairs is not None:      # the pair's length gradient is carried by its representative edge
                    drb = torch.zeros(e, nb, dtype=torch.float32, device=dev).index_copy_(0, pairs[1], drb)
            dsh1 += dsh0
            dvec = self._rows(e, 3)
            _lib.check(lib.ictc_edge_geometry_backward(_lib.ptr(unit), _lib.ptr(length), rmax, nb, pcut, e,
                                                       _lib.ptr(dsh1), _lib.ptr(drb), _lib.ptr(dvec), st),
                       "edge_geometry_backward")
            grad = self._rows(n_local, 3)
            _lib.check(lib.ictc_position_gradient(n_local, n_owned, dst_rowptr.data_ptr(), src_csr[0].data_ptr(),
                                                  _lib.ptr(src_csr[1]), _lib.ptr(dvec), grad.data_ptr(), st),
                       "position_gradient")
        return energy, grad, atomic
