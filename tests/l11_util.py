"""Reader for tests/golden/l11_corpus.txt: the reference's record of all 23 slots of a real W16R2 block core
(grammar: hashline/src/private_block/lean_l11_export_tests.rs:60-262).  Unlike the structural fixture of the recorded
125M graphs, these graphs carry their real coefficient values and each comes with the terminal table values `VALS`
and the reference's own `poly(vals)`, so an evaluator can be held to a number the reference computed."""
import os

P = 0xFFFFFFFF00000001


def _f2s(s):
    if s == "-":
        return []
    w = [int(x) for x in s.split(",")]
    return [(w[i], w[i + 1]) for i in range(0, len(w), 2)]


def _f2(s):
    a, b = s.split(",")
    return (int(a), int(b))


def _coef(s):
    c0, c1, cls = s.split(":")
    return (int(c0), int(c1)), cls


def _factors(s):
    """`t3.n0.n1` -> [("t", 3), ("n", 0), ("n", 1)]"""
    return [] if s == "-" else [(f[0], int(f[1:])) for f in s.split(".")]


def load(golden_dir):
    """{"key": transcript key or None, "head": .., "slots": [..]}"""
    head, slots, cur = {}, [], None
    for line in open(os.path.join(golden_dir, "l11_corpus.txt")):
        w = line.rstrip("\n").split(" ")
        k = w[0]
        if k == "L11":
            head["shape"], head["key"], head["n_slots"] = w[1], (None if w[2] == "-" else bytes.fromhex(w[2])), int(w[3])
        elif k == "HEAD":
            head["head"] = (bytes.fromhex(w[1]), int(w[2]))
        elif k == "ROOTS":
            head["roots"] = dict(a_root=bytes.fromhex(w[1]), a_rows=int(w[2]), mask_root=bytes.fromhex(w[3]), h_root=bytes.fromhex(w[4]),
                                 h_rows=int(w[5]), log_cols=int(w[6]))
        elif k == "LOGUP":
            head["beta"], head["gamma"], head["alpha"] = _f2(w[1]), _f2(w[2]), _f2(w[3])
        elif k == "TAGS":
            head["g_u8"], head["g_exp"], head["g_act"] = _f2(w[1]), _f2(w[2]), _f2(w[3])
        elif k == "HEADEND":
            head["headend"] = (bytes.fromhex(w[1]), int(w[2]))
        elif k == "SLOT":
            cur = dict(slot=int(w[1]), kind=w[2], n=int(w[3]), ext=int(w[4]), degree=int(w[5]), n_priv=int(w[6]), n_tabs=int(w[7]),
                       rounds=[], tabs=[], ir_tabs=[], nodes=[], terms=[])
            slots.append(cur)
        elif k == "DRAWS":
            cur["draws"] = _f2s(w[1])
        elif k == "TRB":
            cur["trb"] = (bytes.fromhex(w[1]), int(w[2]))
        elif k == "TRA":
            cur["tra"] = (bytes.fromhex(w[1]), int(w[2]))
        elif k == "SCALAR":
            cur["scalar"] = _f2(w[1])
        elif k == "HOSTED":
            cur["hosted"] = [] if w[1] == "-" else [(int(h.split(":")[0]), (int(h.split(":")[1]), int(h.split(":")[2]))) for h in w[1].split(";")]
        elif k == "ROUND":
            assert int(w[1]) == len(cur["rounds"])
            cur["rounds"].append(_f2s(w[2]))
        elif k == "TERMS":
            cur["terms_vals"] = _f2s(w[1])
        elif k == "TAB":
            if w[2] == "eq":
                cur["tabs"].append(("eq", int(w[3]), _f2s(w[4])))
            elif w[2] == "pub":
                cur["tabs"].append(("pub", int(w[3]), _f2s(w[4])))
            elif w[2] == "pubv":
                cur["tabs"].append(("pubv", int(w[3]), _f2(w[4])))
            else:
                cur["tabs"].append(("priv", int(w[3])))
        elif k == "VALS":
            cur["vals"] = _f2s(w[1])
        elif k == "IR":
            cur["ir_counts"] = (int(w[1]), int(w[2]), int(w[3]))
        elif k == "IRTAB":
            cur["ir_tabs"].append(w[2])
        elif k == "NODE":
            assert int(w[1]) == len(cur["nodes"])
            if w[2] == "A":
                terms = [] if w[4] == "-" else [(_coef(x.rsplit("@", 1)[0]), int(x.rsplit("@", 1)[1][1:])) for x in w[4].split(";")]
                cur["nodes"].append(("affine", _coef(w[3]), terms))
            else:
                subs = [] if w[3] == "-" else [(_coef(x.rsplit("@", 1)[0]), _factors(x.rsplit("@", 1)[1])) for x in w[3].split(";")]
                cur["nodes"].append(("sum", subs))
        elif k == "TERM":
            wrapper = [] if w[2] == "-" else [int(x) for x in w[2].split(",")]
            cur["terms"].append((_coef(w[1]), wrapper, _factors(w[3])))
        elif k == "RES":
            cur["c"], cur["claimed"], cur["fin"], cur["rho_full"], cur["pv"], cur["g"] = _f2(w[1]), _f2(w[2]), _f2(w[3]), _f2s(w[4]), _f2(w[5]), _f2(w[6])
    assert len(slots) == head["n_slots"]
    return dict(head=head, slots=slots)


def _cw(c, keep_class=True):
    """a recorded coefficient as a SlotProgram coefficient: the special words where the reference marks them, else the value"""
    (v, cls) = c
    if keep_class and cls == "one":
        assert v == (1, 0)
        return "one"
    if keep_class and cls == "neg-one":
        assert v == (P - 1, 0)
        return "neg-one"
    return v


def build_program(backend, slot):
    """(SlotProgram with the RECORDED coefficient values, description for `ir_util.py_eval`)"""
    SP = backend.SlotProgram
    prog = SP(slot["ir_counts"][0])
    desc = {"nodes": [], "terms": []}

    def fw(f):
        return SP.node(f[1]) if f[0] == "n" else f[1]

    for n in slot["nodes"]:
        if n[0] == "affine":
            konst = _cw(n[1])
            terms = [(_cw(c), t) for c, t in n[2]]
            prog.affine(konst, terms)
            desc["nodes"].append(("affine", konst, terms))
        else:
            subs = [(_cw(c), [fw(f) for f in fs]) for c, fs in n[1]]
            prog.sum(subs)
            desc["nodes"].append(("sum", subs))
    for c, wrapper, inner in slot["terms"]:
        prog.term(_cw(c), wrapper, [fw(f) for f in inner])
        desc["terms"].append((_cw(c), list(wrapper) + [fw(f) for f in inner]))
    assert (prog.n_nodes, prog.n_terms) == slot["ir_counts"][1:]
    return prog, desc
