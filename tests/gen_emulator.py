"""NumPy stand-in for the device steps of ``lower_generic.GenProgram`` (test infrastructure only).

Lets the CPU test-suite check the DAG-to-steps lowering against the oracle without a GPU; the
CUDA kernels implement the same step semantics and are checked against the oracle in the GPU tests.
"""
import numpy as np

from ktir_cpu_b200.lower_generic import NP_DT


def _as_compute(x, is_float):
    return x.astype(np.float32) if is_float else x.astype(np.int64)


def _cmp(op, a, b):
    nan = np.isnan(a) | np.isnan(b) if a.dtype.kind == "f" else np.zeros(np.broadcast(a, b).shape, bool)
    base = {"eq": np.equal, "ne": np.not_equal, "lt": np.less, "le": np.less_equal, "gt": np.greater,
            "ge": np.greater_equal}
    if op in ("cmp_ord",):
        return ~nan
    if op == "cmp_uno":
        return nan
    if op == "cmp_true":
        return np.ones(nan.shape, bool)
    if op == "cmp_false":
        return np.zeros(nan.shape, bool)
    if op.endswith("_"):                      # unordered-or forms
        return base[op[5:7]](a, b) | nan
    r = base[op[4:]](a, b)
    return r & ~nan if op != "cmp_ne" or a.dtype.kind != "f" else (r & ~nan)


def run(prog, arena: np.ndarray):
    """Execute ``prog`` on ``arena`` (uint8 array whose offsets are KTIR byte addresses). Returns flags."""
    P = prog.P
    vals = {}
    flags = {"negative_index": False}

    def view(dt):
        return arena.view(NP_DT[dt]) if dt != "i1" else arena

    with np.errstate(all="ignore"):
        for op in prog.ops:
            a = op.attrs
            src = [vals[b.id] for b in op.srcs]
            d = op.dst
            k = op.kind
            if k in ("load", "addr"):
                addr = a["base"][:, None] + a["rel"][None, :]
                if k == "addr":
                    out = addr
                else:
                    mem = view(d.dtype)
                    ok = (addr >= a["lo"]) & (addr < a["hi"])
                    out = np.where(ok, mem[np.where(ok, addr, 0)], 0).astype(NP_DT[d.dtype])
            elif k == "idxadd":
                idx = src[1].astype(np.int64)
                if (idx < 0).any():
                    flags["negative_index"] = True
                out = src[0] + idx * a["stride"]
            elif k == "gather":
                addr = src[0]
                mem = view(d.dtype)
                ok = (addr >= a["lo"]) & (addr < a["hi"])
                out = np.where(ok, mem[np.where(ok, addr, 0)], 0).astype(NP_DT[d.dtype])
            elif k == "constv":
                out = np.broadcast_to(a["table"][None, :], (P, d.elems)).copy()
            elif k == "fill":
                out = np.full((P, 1), a["value"]).astype(NP_DT[d.dtype])
            elif k == "param":
                out = a["values"].reshape(P, 1).astype(NP_DT[d.dtype])
            elif k == "table":
                out = np.asarray(a["values"]).reshape(P, d.elems).astype(NP_DT[d.dtype])
            elif k == "iota":
                shape = a["shape"]
                idx = np.indices(shape)[a["dim"]].reshape(-1)
                out = np.broadcast_to(idx[None, :], (P, d.elems)).astype(np.int64)
            elif k == "map":
                shape = a["shape"]
                if len(shape):
                    grid = np.indices(shape).reshape(len(shape), -1)
                    e = a["offset"] + (np.asarray(a["strides"], np.int64)[:, None] * grid).sum(0)
                else:
                    e = np.array([a["offset"]])
                out = src[0][:, e]
            elif k == "ew":
                out = _ew(a["op"], d.dtype, src, a)
                if out.shape[1] != d.elems:
                    out = np.broadcast_to(out, (P, d.elems)).copy()
            elif k == "redl":
                x = src[0].reshape(P, a["outer"], a["n"], a["inner"])
                h = a["h"]
                lo_, hi_ = x[:, :, :h], x[:, :, h:2 * h]
                comb = _ew(a["op"], d.dtype, [lo_.reshape(P, -1), hi_.reshape(P, -1)], {}).reshape(lo_.shape)
                if a["n"] % 2:
                    comb = np.concatenate([comb, x[:, :, 2 * h:].astype(comb.dtype)], axis=2)
                out = comb.reshape(P, -1)
            elif k == "concat":
                x = np.broadcast_to(src[0], (P, a["outer"] * a["na"] * a["inner"])).reshape(P, a["outer"], a["na"], a["inner"])
                y = np.broadcast_to(src[1], (P, a["outer"] * a["nb"] * a["inner"])).reshape(P, a["outer"], a["nb"], a["inner"])
                out = np.concatenate([x, y], axis=2).reshape(P, -1)
            elif k == "matmul":
                A = src[0].reshape(P, a["batch"], a["M"], a["K"]).astype(np.float32)
                B = src[1].reshape(P, a["batch"], a["K"], a["N"]).astype(np.float32)
                acc = np.zeros((P, a["batch"], a["M"], a["N"]), np.float32)
                for kk in range(a["K"]):
                    acc = acc + A[..., :, kk:kk + 1] * B[..., kk:kk + 1, :]
                out = acc.astype(NP_DT[d.dtype]).reshape(P, -1)
            elif k == "ringred":
                x = src[0].reshape(P, -1)
                out = x.copy()
                srcs = a["sources"]
                if a["cluster"]:
                    # ranks inside the cluster of each point -> points, through the CTA order table
                    order = a["order"]
                    cl = a["cluster"]
                    where = np.empty(P, np.int64)
                    where[order] = np.arange(P)
                    first = (where // cl) * cl
                    srcs = np.where(srcs >= 0, order[np.clip(first[:, None] + srcs, 0, P - 1)], -1)
                for j in range(srcs.shape[1]):
                    live = j < a["counts"]
                    recv = x[np.clip(srcs[:, j], 0, None)]
                    pair = (recv, out) if a["swapped"] else (out, recv)
                    folded = _ew(a["op"], d.dtype, list(pair), {})
                    out = np.where(live[:, None], folded, out)
            elif k == "store":
                addr = a["base"][:, None] + a["rel"][None, :]
                ok = (addr >= a["lo"]) & (addr < a["hi"])
                mem = view(a["dtype"])
                v = np.broadcast_to(src[0], addr.shape)
                mem[addr[ok]] = v[ok]
                continue
            elif k == "scatter":
                addr = src[1]
                mem = view(a["dtype"])
                v = np.broadcast_to(src[0], addr.shape)
                if a.get("any_order"):                  # the lowering promises distinct addresses
                    ok = (addr >= a["lo"]) & (addr < a["hi"])
                    assert len(np.unique(addr[ok])) == int(ok.sum())
                    mem[addr[ok]] = v[ok]
                    continue
                for p in range(P):                      # points in order, elements in order
                    for e in range(addr.shape[1]):
                        t = addr[p, e]
                        if a["lo"] <= t < a["hi"]:
                            mem[t] = v[p, e]
                continue
            else:
                raise NotImplementedError(k)
            vals[d.id] = np.ascontiguousarray(out)
    return flags


def _ew(op, dst_dt, src, attrs):
    any_f = any(s.dtype.kind == "f" for s in src)
    if op == "mov":
        x = src[0]
        if dst_dt in ("f16", "f32"):
            return x.astype(np.float32).astype(NP_DT[dst_dt])
        if x.dtype.kind == "f":
            return np.trunc(x.astype(np.float32)).astype(np.int64).astype(NP_DT[dst_dt])
        return x.astype(np.int64).astype(NP_DT[dst_dt])
    if op == "bitcast":
        x = src[0]
        return x.view(NP_DT[dst_dt]) if x.dtype.itemsize == np.dtype(NP_DT[dst_dt]).itemsize else x.astype(NP_DT[dst_dt])
    if op.startswith("cmp_"):
        is_f = any_f and not attrs.get("cmp_int")
        a, b = (_as_compute(s, is_f) for s in src[:2])
        return _cmp(op, a, b).astype(np.uint8)
    if op == "select":
        c = src[0] != 0
        is_f = dst_dt in ("f16", "f32")
        t, f = (_as_compute(s, is_f) for s in src[1:3])
        return np.where(c, t, f).astype(NP_DT[dst_dt])
    is_f = dst_dt in ("f16", "f32")
    x = [_as_compute(s, is_f) for s in src]
    if is_f:
        one = np.float32(1)
        fn = {"add": lambda: x[0] + x[1], "sub": lambda: x[0] - x[1], "mul": lambda: x[0] * x[1],
              "div": lambda: x[0] / x[1], "rem": lambda: np.fmod(x[0], x[1]),
              # the first operand wins a tie, as in NumPy's half loops (and the device kernels)
              "max": lambda: np.where((x[0] >= x[1]) | np.isnan(x[0]), x[0], x[1]),
              "maxnum": lambda: np.where((x[0] >= x[1]) | np.isnan(x[1]), x[0], x[1]),
              "min": lambda: np.where((x[0] <= x[1]) | np.isnan(x[0]), x[0], x[1]),
              "minnum": lambda: np.where((x[0] <= x[1]) | np.isnan(x[1]), x[0], x[1]),
              "neg": lambda: -x[0], "abs": lambda: np.abs(x[0]), "exp": lambda: np.exp(x[0]),
              "log": lambda: np.log(x[0]), "log2": lambda: np.log2(x[0]), "log1p": lambda: np.log1p(x[0]),
              "sqrt": lambda: np.sqrt(x[0]), "rsqrt": lambda: one / np.sqrt(x[0]), "tanh": lambda: np.tanh(x[0]),
              "sin": lambda: np.sin(x[0]), "cos": lambda: np.cos(x[0]), "ceil": lambda: np.ceil(x[0]),
              "floor": lambda: np.floor(x[0]), "fma": lambda: x[0] * x[1] + x[2],
              "pow": lambda: np.power(x[0], x[1]), "sign": lambda: np.sign(x[0])}[op]
        return fn().astype(np.float32).astype(NP_DT[dst_dt])
    a, b = x[0], (x[1] if len(x) > 1 else None)
    safe = None if b is None else np.where(b == 0, 1, b)
    fn = {"add": lambda: a + b, "sub": lambda: a - b, "mul": lambda: a * b,
          "divf": lambda: a // safe, "divt": lambda: np.trunc(a / safe).astype(np.int64),
          "rem": lambda: a % safe, "remt": lambda: a - np.trunc(a / safe).astype(np.int64) * b,
          "and": lambda: a & b, "or": lambda: a | b, "xor": lambda: a ^ b, "shl": lambda: a << b,
          "shr": lambda: a >> b, "min": lambda: np.minimum(a, b), "max": lambda: np.maximum(a, b),
          "cdiv": lambda: -((-a) // safe), "neg": lambda: -a, "abs": lambda: np.abs(a)}[op]
    return fn().astype(NP_DT[dst_dt])
