"""Force engine: energy and position gradient of the MACE-ICTC model by an explicit forward and reverse
sweep over the B200 kernels, without the autograd tape.

Same arithmetic as ``MaceIctcModel.forward`` followed by ``autograd.grad(E, pos)``
(reference: mace_ictc/hp/runtime.py:82-111 over mace_ictc/models/mace/backbone.py:860-1246), specialised to
what an MD step needs: frozen weights, gradient with respect to positions only.  Every adjoint below is
the hand-written reverse of the line that produced the value; tests compare it with the autograd path.
Node features live in ir_mul rows ([rows, 9C], degree blocks [2l+1, C]) from end to end, so channel
linears are GEMMs over contiguous rows and no mul_ir <-> ir_mul conversion is made.

Gates are streamed (reference: ictc_o3/ops/streamed_gate_message.py:112-116, 193-221; chunk sizes
mace_ictc/interfaces/lammps_hp.py:163-172).  The per-edge gate table [E, P*C] and its gradient are the largest
tensors of the step, so the sweeps can run over chunks of owner rows (``chunk_rows``): the forward produces the
gates of a chunk's edges from the 64-wide hidden state, consumes them and reuses the buffer; the reverse sweep
recomputes the chunk's gates, lets the tensor-product adjoint write the chunk's gate gradients and contracts
them back to the hidden width at once.  No tensor wider than 64 floats per edge outlives a chunk.  Without
chunking the gate table of the (edge, reverse edge) pairs is kept for both sweeps and only the gate gradient is
per edge.  Both modes run the same arithmetic per edge in the same order, so their results agree bit for bit.
"""
from __future__ import annotations

import ctypes as C
import math

import torch

from ictc_o3 import _lib
from ictc_o3.ops.topology import build_csr
from ictc_o3.symmetric_contraction import _ScCall
from .model import SILU_SCALE, MaceIctcModel

_DEGREES = ((0, 1), (1, 3), (4, 5))        # (first component, number of components) of the degree blocks


class ForceEngine:
    """``chunk_rows``: owner rows per chunk of the streamed gate evaluation (None: one pass over everything).
    ``chunk_margin``: a chunk buffer holds ``chunk_rows x mean degree x chunk_margin`` edges; a chunk with more
    edges than that raises ``overflow`` (device flag) and its surplus edges are dropped, never written out of
    bounds.  ``stream_gates``: see the attribute."""

    def __init__(self, model: MaceIctcModel, chunk_rows: int | None = None, chunk_margin: float = 1.3,
                 stream_gates: bool | None = None):
        if len(model.interactions) != 2:
            raise ValueError("the force engine covers the two-interaction model")
        if model.channels != 64:
            raise ValueError("the force engine runs on the 64-channel tensor-core kernels; other widths use the "
                             "autograd route (MolecularDynamics(..., use_engine=False))")
        self.model = model
        self.c = model.channels
        self.dev = next(model.parameters()).device
        self.lib = _lib.load()
        self._versions = None
        self._spec = {0: _lib.tp_spec(0, 2, 2), 1: _lib.tp_spec(2, 2, 2)}
        self.chunk_rows = None if chunk_rows is None else int(chunk_rows)
        self.chunk_margin = float(chunk_margin)
        # with chunks: True = the gates are streamed too (produced per chunk in the forward sweep, recomputed per chunk
        # in the reverse sweep: nothing of size [E, P*C] exists); False = the gate table of the edge pairs is kept whole
        # and only the gate GRADIENT, the largest tensor, lives per chunk (half the GEMM work of streaming);
        # None = keep the table while both layers' tables take less than 40 % of the device memory
        self.stream_gates = stream_gates
        self.overflow = torch.zeros(1, dtype=torch.int32, device=self.dev)   # sticky: a chunk buffer was too small
        self.profile = None      # list of (kernel name, start event, end event) when enabled by a benchmark
        self._bounds = {}
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
            for inter, prod in zip(m.interactions, m.products):
                lin = inter.input_lmax
                fc = [mod.weight.contiguous() for mod in inter.fc if isinstance(mod, torch.nn.Linear)]
                if not (len(fc) == 4 and fc[0].shape[0] == 64 and fc[0].shape[1] <= 8 and tuple(fc[1].shape) == (64, 64)
                        and tuple(fc[2].shape) == (64, 64) and fc[3].shape[1] == 64 and fc[3].shape[0] % 64 == 0):
                    raise ValueError("the force engine needs the radial MLP num_basis (<= 8) -> 64 -> 64 -> 64 -> P*C")
                L = {
                    "up": [inter.linear_up.adapters[str(l)].weight.contiguous() for l in range(lin + 1)],
                    "fc0": fc[0], "nout": fc[3].shape[0],
                    "ml": [(inter.message_linear.weights[str(l)] / max(inter.avg_num_neighbors, 1e-8)).contiguous()
                           for l in range(3)],
                    "counts": [inter.tp.path_counts_by_l[l] for l in range(3)],
                    "tpw": None if bool(torch.all(inter.tp.weight == 1)) else inter.tp.weight.contiguous(),
                    "w3": self._pack(fc[3], 0), "w3t": self._pack(fc[3], 1),
                    "hid": [self._pack(fc[1], 0), self._pack(fc[2], 0)],
                    "hid_t": [self._pack(fc[1], 1), self._pack(fc[2], 1)],
                }
                wsc = inter.self_connection.weights["0"]                                 # [S, C(out), C(in)]
                s = wsc.shape[0]
                L["sc_fwd"] = wsc.permute(2, 0, 1).reshape(c, s * c).contiguous()          # x @ -> [n, S*C(out)]
                L["sc_bwd"] = wsc.permute(1, 0, 2).reshape(c, s * c).contiguous()          # dout @ -> [n, S*C(in)]
                L["bank"] = prod.symmetric_contractions.weight_bank()
                L["target"] = prod.target_lmax
                pl = [(prod.linear[str(l)] / math.sqrt(c)).contiguous() for l in range(prod.target_lmax + 1)]
                L["pl0"], L["pl0_t"] = pl[0], pl[0].t().contiguous()
                # operand-layout copies for the tensor-core channel linears: key -> (packed, k_chunks, n_chunks)
                P = {}
                for l in range(lin + 1):
                    up = L["up"][l]
                    P["up", l] = self._pack_lin(up, up.t().contiguous())                  # x @ up^T
                    P["up_b", l] = self._pack_lin(up.t().contiguous(), up)                # x @ up
                for l in range(3):
                    ml = L["ml"][l]
                    P["ml", l] = self._pack_lin(ml, ml.t().contiguous())                  # x @ ml^T
                    P["ml_b", l] = self._pack_lin(ml.t().contiguous(), ml)                # x @ ml
                for l in range(prod.target_lmax + 1):
                    P["pl", l] = self._pack_lin(pl[l].t().contiguous(), pl[l])            # x @ pl
                    P["pl_b", l] = self._pack_lin(pl[l], pl[l].t().contiguous())          # x @ pl^T
                L["packed"] = P
                self.layers.append(L)
            self.ro0 = m.layer_energy_readouts[0].readout.weight.reshape(-1).contiguous()  # [C]
            self.ro1_w1 = m.last_layer_energy_readout.linear_1.weight.contiguous()          # [16, C]
            self.ro1_w2 = m.last_layer_energy_readout.linear_2.weight.reshape(-1).contiguous()  # [16]
        self._versions = versions

    def _pack(self, w, transpose):
        """A [rows, 64] matrix in the shared-memory operand layout of the tcgen05 kernels."""
        out = torch.empty(2 * w.numel(), dtype=torch.float32, device=w.device)
        with _lib.on_device(w.device):
            _lib.check(self.lib.ictc_gate_pack_weights(w.shape[0], w.data_ptr(), transpose, out.data_ptr(),
                                                       _lib.stream(w.device)), "gate_pack_weights")
        return out

    def _pack_lin(self, w_out_major, w_in_major):
        """Operand copy for out = x @ w_in_major, where w_in_major is [K, N] and w_out_major its transpose."""
        k, n = w_in_major.shape
        if k == 64:
            return self._pack(w_out_major.contiguous(), 0), 1, n // 64
        if n != 64:
            raise ValueError("tensor-core channel linear needs a 64-wide side")
        return self._pack(w_in_major.contiguous(), 1), k // 64, 1

    def _lin(self, L, key, rows, in_t, in_off, in_mm, in_ld, out_t, out_off, out_mm, out_ld):
        """out rows = in rows @ W on the tensor cores, reading / writing per-degree blocks in place."""
        packed, kc, nc = L["packed"][key]
        t0 = self._mark()
        _lib.check(self.lib.ictc_channel_linear_tc(rows, kc, nc, in_t.data_ptr() + 4 * in_off, in_mm, in_ld,
                                                   packed.data_ptr(), out_t.data_ptr() + 4 * out_off, out_mm, out_ld,
                                                   self._st()), "channel_linear_tc")
        self._done("channel_linear_tc", t0)

    def _lin_blocks(self, L, key, rows, in_t, out_t, in_wide=None, out_wide=None, degrees=3):
        """One channel linear per degree block of [rows, 9C] buffers; ``in_wide`` / ``out_wide`` = path-slot counts
        per degree when that side is the [rows, 35C]-style slot-major tensor-product layout."""
        c = self.c
        in_off = out_off = 0
        for l, (off, mm) in enumerate(_DEGREES[:degrees]):
            i_off, i_ld = (in_off, in_t.shape[1]) if in_wide else (off * c, in_t.shape[1])
            o_off, o_ld = (out_off, out_t.shape[1]) if out_wide else (off * c, out_t.shape[1])
            self._lin(L, (key, l), rows * mm, in_t, i_off, mm, i_ld, out_t, o_off, mm, o_ld)
            if in_wide:
                in_off += in_wide[l] * mm * c
            if out_wide:
                out_off += out_wide[l] * mm * c

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

    # ---------------------------------------------------------------- radial MLP
    def _hidden(self, rb, L, rows, count, limit):
        """Hidden layers of the radial MLP: pre-activations z1..z3 [count, 64]; row r reads rb[rows[r]] (rows None:
        rb[r]); ``limit`` = device scalar with the number of rows in use when ``count`` is a capacity."""
        pre = [self._rows(count, 64) for _ in range(3)]
        t0 = self._mark()
        _lib.check(self.lib.ictc_mlp_chain_forward(count, rb.shape[1], _lib.ptr(rb), _lib.ptr(rows), L["fc0"].data_ptr(),
                                                   L["hid"][0].data_ptr(), L["hid"][1].data_ptr(), _lib.ptr(pre[0]),
                                                   _lib.ptr(pre[1]), _lib.ptr(pre[2]), _lib.ptr(limit), self._st()),
                   "mlp_chain_forward")
        self._done(f"radial_mlp_hidden_forward_{L['nout']}", t0)
        return pre

    def _gate_table(self, z3, L, limit):
        """Gates of every row of z3 (one row per edge pair, or per edge without pairing)."""
        count, nout = z3.shape[0], L["nout"]
        gates = self._rows(count, nout)
        t0 = self._mark()
        _lib.check(self.lib.ictc_gate_gemm_forward(count, nout, _lib.ptr(z3), L["w3"].data_ptr(), _lib.ptr(gates), 1,
                                                   _lib.ptr(limit), self._st()), "gate_gemm_forward")
        self._done(f"gate_gemm_forward_{nout}", t0)
        return gates

    def _gate_chunk(self, z3, L, buf, index, begin_ptr, end_ptr):
        """Gates of the list entries [*begin, *end) into ``buf``: row r = act(z3[index[*begin + r]]) @ W3^T."""
        t0 = self._mark()
        _lib.check(self.lib.ictc_gate_gemm_forward_rows(buf.shape[0], L["nout"], _lib.ptr(z3), _lib.ptr(index), begin_ptr,
                                                        end_ptr, L["w3"].data_ptr(), buf.data_ptr(), 1, self._st()),
                   "gate_gemm_forward_rows")
        self._done(f"gate_gemm_forward_{L['nout']}", t0)

    def _streaming(self, table_rows):
        """Are the gates streamed per chunk (True) or is the table of ``table_rows`` rows kept for both sweeps?"""
        if self.stream_gates is not None:
            return bool(self.stream_gates)
        total = torch.cuda.get_device_properties(self.dev).total_memory
        return 4 * table_rows * sum(L["nout"] for L in self.layers) > 0.4 * total

    def _chunks(self, rows, rowptr, edges):
        """[(first row, end row)] of the owner-row chunks and the edge capacity of a chunk buffer; also raises the
        device-side overflow flag when a chunk holds more edges than the buffer."""
        if self.chunk_rows is None or self.chunk_rows >= rows:
            return [(0, rows)], None
        step = self.chunk_rows
        key = (rows, step)
        if key not in self._bounds:        # built outside any stream capture: the first call is a warm-up step
            bounds = list(range(0, rows, step)) + [rows]
            self._bounds[key] = (bounds, torch.tensor(bounds, dtype=torch.int64, device=self.dev))
        bounds, idx = self._bounds[key]
        cap = self.bucket(int(step * (edges / max(rows, 1)) * self.chunk_margin) + 1024)
        cuts = rowptr.index_select(0, idx)
        self.overflow.logical_or_(((cuts[1:] - cuts[:-1]) > cap).any())
        return list(zip(bounds[:-1], bounds[1:])), cap

    # ---------------------------------------------------------------- tensor-product sweeps
    def _tp_forward(self, layer, L, x, sh, z3, src, rowptr, rows, e, grow, limit):
        """Receiver-row sweep of one interaction: gates from z3 (pair rows through ``grow``), message rows out."""
        c, lib = self.c, self.lib
        width = (9 if layer == 0 else 35) * c
        out = self._rows(rows, width)
        chunks, cap = self._chunks(rows, rowptr, e)
        if cap is None or not self._streaming(z3.shape[0]):
            gates = self._gate_table(z3, L, limit)
            t0 = self._mark()
            _lib.check(lib.ictc_tp_graph_forward_shared(self._spec[layer], c, rows, e, x.data_ptr(), sh.data_ptr(),
                                                        _lib.ptr(L["tpw"]), gates.data_ptr(), _lib.ptr(grow),
                                                        src.data_ptr(), rowptr.data_ptr(), None, None, out.data_ptr(),
                                                        self._st()), "tp_graph_forward")
            self._done(f"graph_forward_l{layer}", t0)
            return out, gates
        buf = torch.empty(cap, L["nout"], dtype=torch.float32, device=self.dev)
        for r0, r1 in chunks:
            b, en = rowptr.data_ptr() + 8 * r0, rowptr.data_ptr() + 8 * r1
            self._gate_chunk(z3, L, buf, grow, b, en)
            t0 = self._mark()
            _lib.check(lib.ictc_tp_graph_forward_chunk(self._spec[layer], c, r1 - r0, x.data_ptr(), sh.data_ptr(),
                                                       _lib.ptr(L["tpw"]), buf.data_ptr(), None, b, cap, src.data_ptr(),
                                                       b, None, None, out.data_ptr() + 4 * r0 * width, self._st()),
                       "tp_graph_forward_chunk")
            self._done(f"graph_forward_l{layer}", t0)
        return out, None

    def _tp_adjoint(self, layer, L, x, sh, z3, gates, dst, src_csr, v, n_rows, e, grow, grow_by_pos, need_x):
        """Sender-row sweep: dx [n_rows, .] (optional), dsh [E, 9] and the gradient of silu(z3) per EDGE
        (da3e [E, 64], row = edge id).  The gate gradients exist per chunk only."""
        c, lib = self.c, self.lib
        rowptr, order = src_csr
        nout = L["nout"]
        xw = x.shape[1]
        dx = self._rows(n_rows, xw) if need_x else None
        dsh = self._rows(e, 9)
        da3e = self._rows(e, 64)
        chunks, cap = self._chunks(n_rows, rowptr, e)
        if cap is None:
            cap = self.bucket(max(e, 1))
        table = gates is not None            # the pair table of the forward sweep is still there
        dg = torch.empty(cap, nout, dtype=torch.float32, device=self.dev)
        gbuf = None if table else torch.empty(cap, nout, dtype=torch.float32, device=self.dev)
        for s0, s1 in chunks:
            b, en = rowptr.data_ptr() + 8 * s0, rowptr.data_ptr() + 8 * s1
            if not table:      # the chunk's gates are recomputed for the reverse sweep
                self._gate_chunk(z3, L, gbuf, grow_by_pos, b, en)
            t0 = self._mark()
            _lib.check(lib.ictc_tp_graph_adjoint_chunk(
                self._spec[layer], c, s1 - s0, x.data_ptr() + 4 * s0 * xw, sh.data_ptr(), _lib.ptr(L["tpw"]),
                (gates if table else gbuf).data_ptr(), _lib.ptr(grow) if table else None, 0 if table else 1,
                None if table else b, 0 if table else cap, dst.data_ptr(), b, _lib.ptr(order), None, v.data_ptr(),
                None if dx is None else dx.data_ptr() + 4 * s0 * xw, dsh.data_ptr(), dg.data_ptr(), b, cap, self._st()),
                "tp_graph_adjoint_chunk")
            self._done(f"graph_adjoint_l{layer}", t0)
            t0 = self._mark()
            _lib.check(lib.ictc_gate_gemm_backward_rows(cap, nout, dg.data_ptr(), b, en, _lib.ptr(order),
                                                        L["w3t"].data_ptr(), da3e.data_ptr(), self._st()),
                       "gate_gemm_backward_rows")
            self._done(f"gate_gemm_backward_{nout}", t0)
        return dx, dsh, da3e

    def _hidden_bwd(self, da3e, pre, L, pairs, drb, accumulate, limit):
        """Input gradient of the hidden layers: row u starts from da3e[rep[u]] + da3e[other[u]] (the two edges of a
        pair) and adds / writes its result to drb[rep[u]]; without pairing row = edge."""
        count = pre[0].shape[0]
        pa, pb = (None, None) if pairs is None else (pairs[1], pairs[2])
        t0 = self._mark()
        _lib.check(self.lib.ictc_mlp_chain_backward_paired(
            count, L["fc0"].shape[1], _lib.ptr(da3e), _lib.ptr(pa), _lib.ptr(pb), L["fc0"].data_ptr(),
            L["hid_t"][0].data_ptr(), L["hid_t"][1].data_ptr(), _lib.ptr(pre[0]), _lib.ptr(pre[1]), _lib.ptr(pre[2]),
            _lib.ptr(drb), _lib.ptr(pa), int(accumulate), _lib.ptr(limit), self._st()), "mlp_chain_backward")
        self._done(f"radial_mlp_hidden_backward_{L['nout']}", t0)

    # ---------------------------------------------------------------- the sweep
    @torch.no_grad()
    def energy_and_gradient(self, pos, species, src, dst, shifts, box, n_owned, dst_rowptr, plan=None, n_rows=None,
                            pairs=None, row_mask=None):
        """pos [N_local,3] (owned rows first), species [N_local] (index), edges sorted by receiver with all
        receivers < n_owned, dst_rowptr [n_owned+1].  Returns (energy of owned atoms, dE/dpos [N_local,3],
        per-atom energies [n_owned]).  ``n_rows`` < N_local marks trailing rows of ``pos`` as padding: they may
        be named by inert edges (whose sender index is then outside the sender CSR) but carry no features.
        ``pairs`` = (gate_row [E], rep_edge [U], other_edge [U]) evaluates the radial MLP once per edge pair; an
        optional fourth element is a device int64 scalar with the number of pair rows in use when U is a capacity.
        ``plan`` (an exchange plan of ``mace_ictc.domain``) refreshes the ghost rows between the interactions.
        ``row_mask`` [n_owned] (0 / 1) leaves padding rows among the owned rows out of the energy (and hence of
        the gradient: a padding row has no edges)."""
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
            rep = None if pairs is None else pairs[1]               # the MLP kernels gather / scatter the pair rows
            live = pairs[3] if (pairs is not None and len(pairs) > 3) else None
            count = e if pairs is None else int(rep.numel())
            chunked = (self.chunk_rows is not None and self.chunk_rows < max(n_owned, n_local)
                       and self._streaming(count))
            # gate row of the edge at every position of the sender order (reverse sweep of the streamed mode)
            grow_by_pos = None
            if chunked:
                grow_by_pos = src_csr[1] if grow is None else grow.index_select(0, src_csr[1])
            sp_owned = species[:n_owned]
            s_count = self.emb.shape[0]
            # ---- layer 0
            x0 = self.emb.index_select(0, species)                               # [N_local, C]
            u0 = self._rows(n_local, c)
            self._lin(L0, ("up", 0), n_local, x0, 0, 1, c, u0, 0, 1, c)
            pre0 = self._hidden(rb, L0, rep, count, live)
            M0, g0 = self._tp_forward(0, L0, u0, sh, pre0[2], src, dst_rowptr, n_owned, e, grow, live)   # [n, 9C]
            m0 = self._rows(n_owned, 9 * c)
            self._lin_blocks(L0, "ml", n_owned, M0, m0)
            sc0 = self._species_linear(x0[:n_owned], sp_owned, L0["sc_fwd"], s_count)
            call0 = _ScCall(c, 2, s_count, sp_owned, True)
            y0 = call0.forward(m0, L0["bank"])                                    # [n, 9C]
            h1 = self._rows(n_owned, 9 * c)
            self._lin_blocks(L0, "pl", n_owned, y0, h1)
            h1[:, :c] += sc0
            e0 = torch.mv(h1[:, :c], self.ro0)
            # ---- halo: the ghost rows travel while the layer-1 hidden state (which needs only the radial basis) is computed
            halo = None if plan is None else plan.forward_async(h1)
            pre1 = self._hidden(rb, L1, rep, count, live)
            h1_full = h1 if plan is None else torch.cat((h1, halo()), 0)
            # ---- layer 1
            u1 = self._rows(n_local, 9 * c)
            self._lin_blocks(L1, "up", n_local, h1_full, u1)
            M1, g1 = self._tp_forward(1, L1, u1, sh, pre1[2], src, dst_rowptr, n_owned, e, grow, live)   # [n, 35C]
            m1 = self._rows(n_owned, 9 * c)
            self._lin_blocks(L1, "ml", n_owned, M1, m1, in_wide=L1["counts"])     # slot-major block contracted in place
            del M1
            sc1 = self._species_linear(h1[:, :c].contiguous(), sp_owned, L1["sc_fwd"], s_count)
            call1 = _ScCall(c, 0, s_count, sp_owned, True)
            y1 = call1.forward(m1, L1["bank"])                                    # [n, C]
            h2 = torch.mm(y1, L1["pl0"]) + sc1
            z = torch.mm(h2, self.ro1_w1.t())
            a = self._silu(z)
            e1 = torch.mv(a, self.ro1_w2)
            atomic = e0 + e1
            if row_mask is not None:
                atomic = atomic * row_mask
            energy = atomic.sum()

            # ================= reverse sweep (dE = 1 for every owned atom) =================
            da = self.ro1_w2.unsqueeze(0).expand(n_owned, -1).contiguous()
            if row_mask is not None:
                da = da * row_mask.unsqueeze(1)
            dz = self._silu_bwd(z, da)
            dh2 = torch.mm(dz, self.ro1_w1)                                        # [n, C]
            dy1 = torch.mm(dh2, L1["pl0_t"])
            dm1, _ = call1.adjoint(m1, L1["bank"], dy1, (True, False))             # [n, 9C]
            v1 = self._rows(n_owned, 35 * c)
            self._lin_blocks(L1, "ml_b", n_owned, dm1, v1, out_wide=L1["counts"])
            du1, dsh1, da3e = self._tp_adjoint(1, L1, u1, sh, pre1[2], g1, dst, src_csr, v1, n_local, e, grow,
                                               grow_by_pos, True)
            del v1, g1
            dh1_full = self._rows(n_local, 9 * c)
            self._lin_blocks(L1, "up_b", n_local, du1, dh1_full)
            # the ghost rows' cotangents travel back while the layer-1 MLP is differentiated
            halo = None if plan is None else plan.adjoint_async(dh1_full[n_owned:].contiguous())
            drb = self._rows(e, nb, zero=True)
            self._hidden_bwd(da3e, pre1, L1, pairs, drb, False, live)
            del pre1
            dh1 = dh1_full[:n_owned]
            if plan is not None:
                dh1 = dh1 + halo()
            else:
                dh1 = dh1.clone()
            full = torch.mm(dh2, L1["sc_bwd"]).view(n_owned, s_count, c)
            dh1[:, :c] += full.gather(1, sp_owned.view(-1, 1, 1).expand(-1, 1, c)).squeeze(1)
            dh1[:, :c] += self.ro0 if row_mask is None else self.ro0.unsqueeze(0) * row_mask.unsqueeze(1)
            dy0 = self._rows(n_owned, 9 * c)
            self._lin_blocks(L0, "pl_b", n_owned, dh1, dy0)
            dm0, _ = call0.adjoint(m0, L0["bank"], dy0, (True, False))
            v0 = self._rows(n_owned, 9 * c)
            self._lin_blocks(L0, "ml_b", n_owned, dm0, v0)
            _, dsh0, da3e = self._tp_adjoint(0, L0, u0, sh, pre0[2], g0, dst, src_csr, v0, n_local, e, grow,
                                             grow_by_pos, False)
            self._hidden_bwd(da3e, pre0, L0, pairs, drb, True, live)
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
