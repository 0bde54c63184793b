"""Emit the constant tables of the kernels as C preprocessor X-macro lists.

Reads the host-side plan (``ictc_o3/tables.py``, itself built from ``ictc_tables_lmax2.npz``) and
writes ``generated/tp_spec_tables.cuh``, ``generated/harmonics_tables.cuh`` and
``generated/sc_tables.cuh``.  Every coupling constant becomes a float literal in straight-line
device code, so the sparse Clebsch-Gordan product is a fixed sequence of FMAs with immediate
operands and register-resident operands (no table loads in the inner loop).

Run:  python gen_tables.py     (done by build.py; the outputs are committed so a plain nvcc works)
"""
from __future__ import annotations

import os
import sys

HERE = os.path.dirname(os.path.abspath(__file__))
sys.path.insert(0, os.path.dirname(HERE))

from ictc_o3 import tables as T  # noqa: E402

# (input_lmax, edge_lmax, output_lmax) path sets that get compiled kernels
TP_SPECS = [(0, 0, 0), (0, 1, 1), (1, 1, 1), (0, 2, 2), (2, 2, 2), (2, 2, 0)]


def flit(v: float) -> str:
    s = repr(float(v))
    if "e" not in s and "." not in s and "inf" not in s:
        s += ".0"
    return s + "f"


def spec_name(spec):
    return "L%d%d%d" % spec


def emit_tp(lines):
    lines.append("// (i,j,k,p,c): out comp k of path p gets c * x[i] * sh[j].  F = first term of its group, A = accumulate.")
    for sid, spec in enumerate(TP_SPECS):
        lin, ledge, lout = spec
        plan = T.tp_plan(tuple(T.natural_paths(*spec)), lin, ledge, max(spec))
        n = spec_name(spec)
        lines.append(f"// ---- spec {n}: paths {list(plan.paths)}")
        lines.append(f"#define ICTC_TP_{n}_ID {sid}")
        for key, val in (("NX", plan.nx), ("NH", plan.nh), ("NP", plan.num_paths), ("NO", plan.no),
                         ("NNZ", len(plan.nnz))):
            lines.append(f"#define ICTC_TP_{n}_{key} {val}")
        # (i,p) groups for the adjoint: q index
        qs = sorted({(i, p) for i, _j, _k, p, _c in plan.nnz})
        qidx = {ip: q for q, ip in enumerate(qs)}
        lines.append(f"#define ICTC_TP_{n}_NQ {len(qs)}")

        def lst(name, entries, keyf, fmt):
            out, seen = [], set()
            for ent in sorted(entries, key=keyf):
                kind = "A" if keyf(ent)[0] in seen else "F"
                seen.add(keyf(ent)[0])
                out.append(f"{kind}({fmt(ent)})")
            lines.append(f"#define ICTC_TP_{n}_{name}(F,A) \\\n  " + " \\\n  ".join(
                " ".join(out[a:a + 4]) for a in range(0, len(out), 4)))

        full = lambda e: f"{e[0]},{e[1]},{e[2]},{e[3]},{flit(e[4])}"
        lst("BYK", plan.nnz, lambda e: (e[2], e[0], e[1]), full)
        lst("BYJ", plan.nnz, lambda e: (e[1], e[2], e[0]), full)
        lst("BYQ", plan.nnz, lambda e: (qidx[(e[0], e[3])], e[1], e[2]),
            lambda e: f"{qidx[(e[0], e[3])]},{e[1]},{e[2]},{flit(e[4])}")
        lines.append(f"#define ICTC_TP_{n}_QLIST(X) " + " ".join(f"X({q},{i},{p})" for q, (i, p) in enumerate(qs)))
        # dx[i] accumulates over its q groups: first/accumulate by i
        seen, ent = set(), []
        for q, (i, p) in enumerate(qs):
            ent.append(f"{'A' if i in seen else 'F'}({q},{i},{p})")
            seen.add(i)
        lines.append(f"#define ICTC_TP_{n}_QBYI(F,A) " + " ".join(ent))
        seen, ent = set(), []
        for q, (i, p) in sorted(enumerate(qs), key=lambda t: (t[1][1], t[1][0])):
            ent.append(f"{'A' if p in seen else 'F'}({q},{i},{p})")
            seen.add(p)
        lines.append(f"#define ICTC_TP_{n}_QBYP(F,A) " + " ".join(ent))
        op = plan.out_path()
        lines.append(f"#define ICTC_TP_{n}_OUTP(X) " + " ".join(f"X({k},{p})" for k, p in enumerate(op)))
        # ---- per-edge geometry b[i,k] = sum_j C[i,j,k] sh[j] (at most two terms per entry) shared by all
        # channels of an edge.  FB: entries ordered for the forward (by output k), AB: for the adjoint
        # (by (i,p) group).  *_TAB(X): X(j1, c1, j2, c2) rows used to build b from the harmonics.
        ik = {}
        for i, j, k, p_, c in plan.nnz:
            ik.setdefault((i, k, p_), []).append((j, c))
        assert max(len(v) for v in ik.values()) <= 2
        lines.append(f"#define ICTC_TP_{n}_NB {len(ik)}")

        def btab(name, order):
            rows = []
            for key in order:
                terms = ik[key] + [(0, 0.0)]
                rows.append(f"X({terms[0][0]},{flit(terms[0][1])},{terms[1][0]},{flit(terms[1][1])})")
            lines.append(f"#define ICTC_TP_{n}_{name}_TAB(X) \\\n  " + " \\\n  ".join(
                " ".join(rows[a:a + 4]) for a in range(0, len(rows), 4)))

        fb = sorted(ik, key=lambda t: (t[1], t[0]))
        btab("FB", fb)
        seen, ent = set(), []
        for e, (i, k, p_) in enumerate(fb):
            ent.append(f"{'A' if k in seen else 'F'}({e},{i})")
            seen.add(k)
            if e + 1 == len(fb) or fb[e + 1][1] != k:
                ent.append(f"K({k},{p_})")
        lines.append(f"#define ICTC_TP_{n}_FB(F,A,K) \\\n  " + " \\\n  ".join(
            " ".join(ent[a:a + 6]) for a in range(0, len(ent), 6)))
        ab = sorted(ik, key=lambda t: (qidx[(t[0], t[2])], t[1]))
        btab("AB", ab)
        ent = []
        for e, (i, k, p_) in enumerate(ab):
            first = e == 0 or qidx[(ab[e - 1][0], ab[e - 1][2])] != qidx[(i, p_)]
            last = e + 1 == len(ab) or qidx[(ab[e + 1][0], ab[e + 1][2])] != qidx[(i, p_)]
            ent.append(f"{'F' if first else 'A'}({e},{k})")
            if last:
                ent.append(f"Q({i},{p_})")
        lines.append(f"#define ICTC_TP_{n}_AB(F,A,Q) \\\n  " + " \\\n  ".join(
            " ".join(ent[a:a + 6]) for a in range(0, len(ent), 6)))
        # couplings ordered by harmonic j with their position t in the constant array
        byj = sorted(plan.nnz, key=lambda e_: (e_[1], e_[2], e_[0]))
        lines.append(f"#define ICTC_TP_{n}_CLIST(X) " + " ".join(f"X({flit(e_[4])})" for e_ in byj))
        import struct
        bits = [struct.unpack("<I", struct.pack("<f", e_[4]))[0] for e_ in byj]
        lines.append(f"#define ICTC_TP_{n}_CLIST64(X) " + " ".join(f"X(0x{b:08x}{b:08x}ULL)" for b in bits))
        seen, ent = set(), []
        for t, (i, j, k, p_, c) in enumerate(byj):
            ent.append(f"{'A' if j in seen else 'F'}({t},{i},{j},{k},{p_})")
            seen.add(j)
        lines.append(f"#define ICTC_TP_{n}_BYJT(F,A) \\\n  " + " \\\n  ".join(
            " ".join(ent[a:a + 5]) for a in range(0, len(ent), 5)))
        # ---- path-major program of the fused adjoint: per path p the cotangent slots of p are loaded (VL), every
        # (i,p) group contracts geometry with them (ZF/ZA, then Q: dx[i] and the gate gradient of p), the slots are
        # gated (VG) and the literal couplings of p give the harmonic gradient (DS: t = position in CLIST).  Only
        # the slots of a few paths are live at a time (loads run two paths ahead of their use).  AP_TAB: geometry rows in
        # this program's order.
        ap = sorted(ik, key=lambda t: (t[2], t[0], t[1]))
        btab("AP", ap)
        pos_t = {(i, j, k, p_): t for t, (i, j, k, p_, c) in enumerate(byj)}
        ent = []
        ahead = 99                         # cotangent slots are requested this many paths before their use
        slots_of = [[k for k, pp in enumerate(op) if pp == q_] for q_ in range(plan.num_paths)]
        for q_ in range(min(ahead, plan.num_paths)):
            ent += [f"VL({k})" for k in slots_of[q_]]
        for p_ in range(plan.num_paths):
            slots = slots_of[p_]
            ent.append(f"PB({p_})")
            if p_ + ahead < plan.num_paths:
                ent += [f"VL({k})" for k in slots_of[p_ + ahead]]
            rows = [(e, t) for e, t in enumerate(ap) if t[2] == p_]
            for n_, (e, (i, k, _pp)) in enumerate(rows):
                first = n_ == 0 or rows[n_ - 1][1][0] != i
                last = n_ + 1 == len(rows) or rows[n_ + 1][1][0] != i
                ent.append(f"{'ZF' if first else 'ZA'}({e},{k})")
                if last:
                    ent.append(f"Q({i},{p_})")
            ent += [f"VG({k},{p_})" for k in slots]
            # couplings of the path ordered by (slot, input component): consecutive terms feed different harmonic
            # accumulators, so their FMAs do not wait for one another
            # couplings of the path grouped by (harmonic j, coupling value): the products x[i] * vg[k] of a group are
            # summed first (DF opens the group, DA adds to it) and the group meets its coupling once (DE: t = position
            # of one member in CLIST)
            groups = {}
            for (i, j, k, pp, c) in sorted((e_ for e_ in plan.nnz if e_[3] == p_), key=lambda e_: (e_[2], e_[0], e_[1])):
                groups.setdefault((j, struct.pack("<f", c)), []).append((i, k, pos_t[(i, j, k, pp)]))
            for (j, _c), members in groups.items():
                for m_, (i, k, t) in enumerate(members):
                    ent.append(f"{'DF' if m_ == 0 else 'DA'}({i},{k})")
                ent.append(f"DE({members[0][2]},{j})")
            ent.append(f"PE({p_})")
        lines.append(f"#define ICTC_TP_{n}_ADJP(PB,VL,ZF,ZA,Q,VG,DF,DA,DE,PE) \\\n  " + " \\\n  ".join(
            " ".join(ent[a:a + 6]) for a in range(0, len(ent), 6)))
        used_i = sorted({e[0] for e in plan.nnz})
        used_j = sorted({e[1] for e in plan.nnz})
        lines.append(f"#define ICTC_TP_{n}_XUSED(X) " + " ".join(f"X({i})" for i in used_i))
        lines.append(f"#define ICTC_TP_{n}_HUSED(X) " + " ".join(f"X({j})" for j in used_j))
        lines.append("")
    lines.append("#define ICTC_TP_SPEC_LIST(X) " + " ".join(
        f"X({spec_name(s)},{s[0]},{s[1]},{s[2]})" for s in TP_SPECS))


def emit_harmonics(lines):
    terms = T.harmonic_terms(T.TABLE_LMAX)
    lines.append("// T(h, a, b, c, coeff):  Y[h] += coeff * x^a y^b z^c   (flat harmonic index h, degrees ascending)")
    lines.append("#define ICTC_HARM_LMAX %d" % T.TABLE_LMAX)
    ent = []
    for h, rows in enumerate(terms):
        for (a, b, c), v in rows:
            ent.append(f"T({h},{a},{b},{c},{flit(v)})")
    lines.append("#define ICTC_HARM_TERMS(T) \\\n  " + " \\\n  ".join(" ".join(ent[a:a + 3]) for a in range(0, len(ent), 3)))


def write(name, emit):
    lines = ["// GENERATED by gen_tables.py from ictc_tables_lmax2.npz -- do not edit.", "#pragma once", ""]
    emit(lines)
    path = os.path.join(HERE, "generated", name)
    text = "\n".join(lines) + "\n"
    if not os.path.exists(path) or open(path).read() != text:
        with open(path, "w") as f:
            f.write(text)
    return path


def main():
    write("tp_spec_tables.cuh", emit_tp)
    write("harmonics_tables.cuh", emit_harmonics)


# ------------------------------------------------------------------------------------------------
# Symmetric contraction (correlation 3, lmax 2): straight-line polynomial code.
#
# y[l,m] = sum_nu sum_p W[l,nu,p] * sum_{monomials} A[l,nu][m, monomial, p] * monomial(x), where A is the
# U tensor of the reference symmetrised over the feature indices (x (x) x (x) x is symmetric, so only
# the symmetric part of U contributes).  Code is emitted for a generic number type T so the same text
# serves plain floats and first-order dual numbers (for mixed second derivatives).
def sc_coefficients():
    import itertools
    import numpy as np
    out = {}
    for l in range(T.TABLE_LMAX + 1):
        for nu in (1, 2, 3):
            u = T.sc_u_tensor(l, nu)
            if l == 0:
                u = u[None]
            sym = {}
            for idx in itertools.product(range(u.shape[1]), repeat=nu):
                key = tuple(sorted(idx))
                sym[key] = sym.get(key, 0) + u[(slice(None),) + idx]
            terms = {}   # (p, m) -> [(monomial, coeff)]
            for key, blk in sorted(sym.items()):
                for m in range(blk.shape[0]):
                    for p in range(blk.shape[1]):
                        if abs(blk[m, p]) > T.COEFF_THRESHOLD:
                            terms.setdefault((p, m), []).append((key, float(blk[m, p])))
            out[(l, nu)] = (u.shape[-1], terms)
    return out


def sc_weight_offsets(target_lmax):
    """Offset of the (l_out, nu) weight block inside the packed per-species bank; order (l, nu, p)."""
    coefs = sc_coefficients()
    off, res = 0, {}
    for l in range(target_lmax + 1):
        for nu in (1, 2, 3):
            res[(l, nu)] = off
            off += coefs[(l, nu)][0]
    return res, off


def _mono_expr(key):
    if len(key) == 1:
        return f"x[{key[0]}]"
    if len(key) == 2:
        return f"q{key[0]}{key[1]}"
    return f"mul(q{key[0]}{key[1]}, x[{key[2]}])"


def emit_sc(lines):
    coefs = sc_coefficients()
    lines.append("// Symmetric contraction, lmax 2, correlation 3.  LT = target lmax (0 or 2).")
    lines.append("// Number type T needs: mul(T,T), add(T,T), madd(float,T,T) = c*a+b, fmadd(T,T,T) = a*b+c, scale(float,T), zero<T>().")
    for lt in (0, T.TABLE_LMAX):
        woff, nw = sc_weight_offsets(lt)
        lines.append(f"#define ICTC_SC_NW_LT{lt} {nw}")
    quad = [(a, b) for a in range(9) for b in range(a, 9)]

    def used_quads(ls):
        used = set()
        for l in ls:
            for nu in (2, 3):
                for tl in coefs[(l, nu)][1].values():
                    for key, _c in tl:
                        used.add((key[0], key[1]))
        return sorted(used)

    for lt in (0, T.TABLE_LMAX):
        ls = list(range(lt + 1))
        woff, nw = sc_weight_offsets(lt)
        qs = used_quads(ls)
        # ---------------- forward
        lines.append(f"template <class T, class WF> __device__ __forceinline__ void sc_forward_lt{lt}(const T (&x)[9], WF w, T (&y)[{(lt + 1) ** 2}]) {{")
        for a, b in qs:
            lines.append(f"  const T q{a}{b} = mul(x[{a}], x[{b}]);")
        for l in ls:
            for m in range(2 * l + 1):
                lines.append(f"  y[{l * l + m}] = zero<T>();")
            for nu in (1, 2, 3):
                npath, terms = coefs[(l, nu)]
                for p in range(npath):
                    ms = [m for m in range(2 * l + 1) if (p, m) in terms]
                    if not ms:
                        continue
                    lines.append(f"  {{ const T wp = w({woff[(l, nu)] + p});")
                    for m in ms:
                        tl = terms[(p, m)]
                        lines.append(f"    {{ T t = scale({flit(tl[0][1])}, {_mono_expr(tl[0][0])});")
                        for key, c in tl[1:]:
                            lines.append(f"      t = madd({flit(c)}, {_mono_expr(key)}, t);")
                        lines.append(f"      y[{l * l + m}] = fmadd(wp, t, y[{l * l + m}]); }}")
                    lines.append("  }")
        lines.append("}")
        # ---------------- weight gradient: gw[idx] = sum_m gy[l,m] * t[l,nu,p,m]
        lines.append(f"template <class T, class GF> __device__ __forceinline__ void sc_wgrad_lt{lt}(const T (&x)[9], const T (&gy)[{(lt + 1) ** 2}], GF gw) {{")
        for a, b in qs:
            lines.append(f"  const T q{a}{b} = mul(x[{a}], x[{b}]);")
        for l in ls:
            for nu in (1, 2, 3):
                npath, terms = coefs[(l, nu)]
                for p in range(npath):
                    ms = [m for m in range(2 * l + 1) if (p, m) in terms]
                    if not ms:
                        lines.append(f"  gw({woff[(l, nu)] + p}, zero<T>());")
                        continue
                    lines.append("  { T acc = zero<T>();")
                    for m in ms:
                        tl = terms[(p, m)]
                        lines.append(f"    {{ T t = scale({flit(tl[0][1])}, {_mono_expr(tl[0][0])});")
                        for key, c in tl[1:]:
                            lines.append(f"      t = madd({flit(c)}, {_mono_expr(key)}, t);")
                        lines.append(f"      acc = fmadd(gy[{l * l + m}], t, acc); }}")
                    lines.append(f"    gw({woff[(l, nu)] + p}, acc); }}")
        lines.append("}")
        # ---------------- feature gradient: gx = d<gy, y>/dx, one output degree at a time
        lines.append(f"template <class T, class WF> __device__ __forceinline__ void sc_xgrad_lt{lt}(const T (&x)[9], WF w, const T (&gy)[{(lt + 1) ** 2}], T (&gx)[9]) {{")
        for a, b in qs:
            lines.append(f"  const T q{a}{b} = mul(x[{a}], x[{b}]);")
        for i in range(9):
            lines.append(f"  gx[{i}] = zero<T>();")
        for l in ls:
            lines.append("  {")
            bymono = {}
            for nu in (1, 2, 3):
                npath, terms = coefs[(l, nu)]
                for (p, m), tl in sorted(terms.items()):
                    for key, c in tl:
                        bymono.setdefault(key, []).append((nu, p, m, c))
            used_a = sorted({(nu, p, m) for v in bymono.values() for nu, p, m, _c in v})
            for nu, p, m in used_a:
                lines.append(f"    const T a{nu}_{p}_{m} = mul(w({woff[(l, nu)] + p}), gy[{l * l + m}]);")
            for key, tl in sorted(bymono.items(), key=lambda kv: (len(kv[0]), kv[0])):
                nu, p, m, c = tl[0]
                lines.append(f"    {{ T g = scale({flit(c)}, a{nu}_{p}_{m});")
                for nu, p, m, c in tl[1:]:
                    lines.append(f"      g = madd({flit(c)}, a{nu}_{p}_{m}, g);")
                if len(key) == 1:
                    lines.append(f"      gx[{key[0]}] = add(gx[{key[0]}], g); }}")
                elif len(key) == 2:
                    a, b = key
                    if a == b:
                        lines.append(f"      gx[{a}] = fmadd(g, add(x[{a}], x[{a}]), gx[{a}]); }}")
                    else:
                        lines.append(f"      gx[{a}] = fmadd(g, x[{b}], gx[{a}]); gx[{b}] = fmadd(g, x[{a}], gx[{b}]); }}")
                else:
                    a, b, c3 = key
                    # d(x_a x_b x_c): group equal indices
                    from collections import Counter
                    cnt = Counter(key)
                    stmts = []
                    for v, mult in sorted(cnt.items()):
                        rest = list(key)
                        rest.remove(v)
                        r0, r1 = sorted(rest)
                        qn = f"q{r0}{r1}" if (r0, r1) in set(qs) else f"mul(x[{r0}], x[{r1}])"
                        gterm = "g" if mult == 1 else f"scale({float(mult)}f, g)"
                        stmts.append(f"gx[{v}] = fmadd({gterm}, {qn}, gx[{v}]);")
                    lines.append("      " + " ".join(stmts) + " }")
            lines.append("  }")
        lines.append("}")
        lines.append("")


_main_tp = main


def main():  # noqa: F811
    _main_tp()
    write("sc_code.cuh", emit_sc)


if __name__ == "__main__":
    main()
