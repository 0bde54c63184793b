"""The straight-line programs the TP kernels are generated from (csrc/generated/tp_spec_tables.cuh), interpreted in
numpy: the forward program (per-edge geometry entries + gated accumulation), the adjoint-by-group program and the
path-major fused adjoint (geometry contraction, gate gradient, grouped harmonic-gradient couplings) must be
algebraically equal to the plain coupling list out[k] += C[i,j,k] x[i] sh[j] g[p(k)] of the same header
(reference semantics: ictc_o3/backends/k100/generated_cartesian_message.py:120-225, one term per nonzero coupling)."""
import os
import re

import numpy as np
import pytest

HEADER = os.path.join(os.path.dirname(os.path.abspath(__file__)), "..", "ictc-o3-hp-k100_b200", "csrc", "generated",
                      "tp_spec_tables.cuh")


def _macros():
    text = open(HEADER).read().replace("\\\n", " ")
    out = {}
    for m in re.finditer(r"#define (ICTC_TP_\w+?)(\(([\w,]*)\))? (.*)", text):
        out[m.group(1)] = m.group(4).strip()
    return out


def _calls(body):
    """[(macro letter(s), [numbers])] of a list like 'F(0,1,2.5f) A(3,4)'."""
    res = []
    for name, args in re.findall(r"(\w+)\(([^()]*)\)", body):
        vals = [float(a.rstrip("fULL")) if not a.startswith("0x") else int(a.rstrip("UL"), 16) for a in args.split(",") if a]
        res.append((name, vals))
    return res


SPECS = ["L000", "L011", "L111", "L022", "L222", "L220"]


@pytest.mark.parametrize("spec", SPECS)
def test_generated_programs_equal_the_coupling_list(spec):
    mac = _macros()
    g = lambda key: mac[f"ICTC_TP_{spec}_{key}"]
    nx, nh, np_, no, nb = (int(g(k)) for k in ("NX", "NH", "NP", "NO", "NB"))
    terms = [(int(a[0]), int(a[1]), int(a[2]), int(a[3]), a[4]) for _n, a in _calls(g("BYK"))]     # (i, j, k, p, c)
    assert len(terms) == int(g("NNZ"))
    rng = np.random.default_rng(abs(hash(spec)) % 1000)
    x, sh, gate, v = rng.normal(size=nx), rng.normal(size=nh), rng.normal(size=np_), rng.normal(size=no)
    # ---- plain coupling list: value and the three first derivatives contracted with the cotangent v
    out = np.zeros(no)
    dx, dsh, dg = np.zeros(nx), np.zeros(nh), np.zeros(np_)
    for i, j, k, p, c in terms:
        out[k] += c * x[i] * sh[j] * gate[p]
        dx[i] += c * sh[j] * gate[p] * v[k]
        dsh[j] += c * x[i] * gate[p] * v[k]
        dg[p] += c * x[i] * sh[j] * v[k]

    def geometry(tab):
        rows = [a for _n, a in _calls(g(tab))]
        assert len(rows) == nb
        return np.array([c1 * sh[int(j1)] + c2 * sh[int(j2)] for j1, c1, j2, c2 in rows])

    # ---- forward program: t = sum_e b[e] x[i];  acc[k] += t * gate[p]
    b = geometry("FB_TAB")
    acc, t = np.zeros(no), 0.0
    for name, a in _calls(g("FB")):
        if name == "F":
            t = x[int(a[1])] * b[int(a[0])]
        elif name == "A":
            t += x[int(a[1])] * b[int(a[0])]
        else:
            acc[int(a[0])] += t * gate[int(a[1])]
    np.testing.assert_allclose(acc, out, rtol=1e-12, atol=1e-13)
    # ---- adjoint by (i, p) group: z = sum_e b[e] v[k];  dx[i] += z gate[p];  dg[p] += x[i] z
    b = geometry("AB_TAB")
    dx2, dg2, z = np.zeros(nx), np.zeros(np_), 0.0
    for name, a in _calls(g("AB")):
        if name == "F":
            z = b[int(a[0])] * v[int(a[1])]
        elif name == "A":
            z += b[int(a[0])] * v[int(a[1])]
        else:
            dx2[int(a[0])] += z * gate[int(a[1])]
            dg2[int(a[1])] += x[int(a[0])] * z
    np.testing.assert_allclose(dx2, dx, rtol=1e-12, atol=1e-13)
    np.testing.assert_allclose(dg2, dg, rtol=1e-12, atol=1e-13)
    # ---- path-major fused adjoint with grouped couplings
    b = geometry("AP_TAB")
    consts = [a[0] for _n, a in _calls(g("CLIST"))]
    dx3, dg3, dsh3 = np.zeros(nx), np.zeros(np_), np.zeros(nh)
    vv, vg = np.full(no, np.nan), np.full(no, np.nan)
    z = gp = dgp = s = 0.0
    for name, a in _calls(g("ADJP")):
        a = [int(q) for q in a]
        if name == "VL":
            vv[a[0]] = v[a[0]]
        elif name == "PB":
            gp, dgp = gate[a[0]], 0.0
        elif name == "ZF":
            z = b[a[0]] * vv[a[1]]
        elif name == "ZA":
            z += b[a[0]] * vv[a[1]]
        elif name == "Q":
            dx3[a[0]] += z * gp
            dgp += x[a[0]] * z
        elif name == "VG":
            vg[a[0]] = vv[a[0]] * gp
        elif name == "DF":
            s = x[a[0]] * vg[a[1]]
        elif name == "DA":
            s += x[a[0]] * vg[a[1]]
        elif name == "DE":
            dsh3[a[1]] += s * consts[a[0]]
        elif name == "PE":
            dg3[a[0]] = dgp
        else:
            raise AssertionError(name)
    np.testing.assert_allclose(dx3, dx, rtol=1e-12, atol=1e-13)
    np.testing.assert_allclose(dg3, dg, rtol=1e-12, atol=1e-13)
    np.testing.assert_allclose(dsh3, dsh, rtol=1e-6, atol=1e-7)      # the constants are float32 literals of one group member


@pytest.mark.parametrize("name,spec", [("tp_c5_l111_e13_w", "L111"), ("tp_c8_l022_e19", "L022"), ("tp_c8_l222_e37", "L222")])
def test_generated_coupling_list_matches_reference_outputs(name, spec):
    """The coupling list of the generated header, evaluated in numpy on the inputs of the reference-produced vectors
    (tests/golden/make_golden.py: the reference's own EdgeTensorProduct), gives the reference's outputs: the constants
    the kernels are compiled from are pinned on the reference without a GPU."""
    mac = _macros()
    gold = np.load(os.path.join(os.path.dirname(HEADER), "..", "..", "..", "tests", "golden", name + ".npz"))
    lin, lout, c = int(gold["lin"]), int(gold["lout"]), int(gold["channels"])
    paths = [tuple(int(v) for v in p) for p in gold["paths"]]
    e = gold["sh"].shape[0]
    x = np.concatenate([np.transpose(gold[f"x{l}"], (0, 2, 1)) for l in range(lin + 1)], axis=1)      # [E, i, C]
    sh = gold["sh"]
    gates = gold["gates"].reshape(e, len(paths), c) * gold["weight"][None]
    terms = [(int(a[0]), int(a[1]), int(a[2]), int(a[3]), a[4]) for _n, a in _calls(mac[f"ICTC_TP_{spec}_BYK"])]
    outp = {int(a[0]): int(a[1]) for _n, a in _calls(mac[f"ICTC_TP_{spec}_OUTP"])}
    no = int(mac[f"ICTC_TP_{spec}_NO"])
    out = np.zeros((e, no, c))
    for i, j, k, p, coef in terms:
        assert outp[k] == p
        out[:, k] += coef * x[:, i] * sh[:, j, None] * gates[:, p]
    # output slots: degree -> path slot (paths of that output degree, in path order) -> component
    k = 0
    for l in range(lout + 1):
        slots = [p for p, (_a, _b, lo) in enumerate(paths) if lo == l]
        ref = gold[f"out{l}"].reshape(e, len(slots), c, 2 * l + 1)
        for s, p in enumerate(slots):
            for m in range(2 * l + 1):
                assert outp[k] == p
                err = np.abs(out[:, k] - ref[:, s, :, m]).max()
                assert err <= 3e-7 * max(np.abs(ref).max(), 1e-30), (l, s, m, err)
                k += 1
    assert k == no


def test_generated_harmonic_polynomials_match_reference_harmonics():
    """The polynomial table the harmonics kernels are compiled from (csrc/generated/harmonics_tables.cuh), evaluated in
    numpy on the unit vectors of the reference-produced harmonics vectors: values and the gradient contracted with the
    stored cotangent (the table is differentiated term by term, as the kernel does)."""
    text = open(os.path.join(os.path.dirname(HEADER), "harmonics_tables.cuh")).read().replace("\\\n", " ")
    body = re.search(r"#define ICTC_HARM_TERMS\(T\) (.*)", text).group(1)
    terms = [(int(a[0]), int(a[1]), int(a[2]), int(a[3]), a[4]) for _n, a in _calls(body)]
    gold = np.load(os.path.join(os.path.dirname(HEADER), "..", "..", "..", "tests", "golden", "harmonics_l2_e41.npz"))
    n, cot = gold["n"], gold["cot"]
    y, dn = np.zeros_like(gold["y"]), np.zeros_like(n)
    for h, a, b, c, coef in terms:
        px, py, pz = n[:, 0] ** a, n[:, 1] ** b, n[:, 2] ** c
        y[:, h] += coef * px * py * pz
        if a:
            dn[:, 0] += cot[:, h] * coef * a * n[:, 0] ** (a - 1) * py * pz
        if b:
            dn[:, 1] += cot[:, h] * coef * b * px * n[:, 1] ** (b - 1) * pz
        if c:
            dn[:, 2] += cot[:, h] * coef * c * px * py * n[:, 2] ** (c - 1)
    assert np.abs(y - gold["y"]).max() <= 3e-7 * np.abs(gold["y"]).max()
    assert np.abs(dn - gold["dn"]).max() <= 3e-7 * np.abs(gold["dn"]).max()
