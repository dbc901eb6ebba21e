"""KTIR source generators for the benchmark workloads.

The reference ships its kernels as ``.mlir`` examples and notebook templates
(examples/triton-ktir/*.mlir, notebooks/demo_gen_mlir.py:109-218); the sizes the
benchmarks need do not exist as files there, so the text is produced here.
Every generator returns a complete ``module { func.func ... }`` string that both
this backend and the reference interpreter accept.
"""
from __future__ import annotations

from typing import Sequence


def _box(shape: Sequence[int]) -> str:
    dims = ", ".join(f"d{i}" for i in range(len(shape)))
    cons = ", ".join(f"d{i} >= 0, -d{i} + {s - 1} >= 0" for i, s in enumerate(shape))
    return f"affine_set<({dims}) : ({cons})>"


def _ident(n: int) -> str:
    dims = ", ".join(f"d{i}" for i in range(n))
    return f"affine_map<({dims}) -> ({dims})>"


def _xs(shape: Sequence[int], dtype: str) -> str:
    return "x".join(str(s) for s in shape) + "x" + dtype


def _rowmajor(shape: Sequence[int]):
    st, acc = [], 1
    for s in reversed(shape):
        st.append(acc)
        acc *= s
    return list(reversed(st))


def view(name: str, ptr: str, shape: Sequence[int], dtype: str, strides=None) -> str:
    strides = strides or _rowmajor(shape)
    return (f"    %{name} = ktdp.construct_memory_view %{ptr}, sizes: {list(shape)}, strides: {list(strides)} {{\n"
            f"      coordinate_set = {_box(shape)}, memory_space = #ktdp.memory_space<global>\n"
            f"    }} : memref<{_xs(shape, dtype)}>\n")


def tile(name: str, vw: str, idx: Sequence[str], tshape: Sequence[int], vshape: Sequence[int],
         dtype: str, indent: str = "    ") -> str:
    return (f"{indent}%{name} = ktdp.construct_access_tile %{vw}[{', '.join(idx)}] {{\n"
            f"{indent}  access_tile_set = {_box(tshape)},\n"
            f"{indent}  access_tile_order = {_ident(len(tshape))}\n"
            f"{indent}}} : memref<{_xs(vshape, dtype)}> -> !ktdp.access_tile<{_xs(tshape, 'index')}>\n")


def vector_add(n: int = 4096, block: int = 128, cores: int = 32, dtype: str = "f16") -> str:
    """out = x + y; core c adds blocks c, c + cores, ... of ``block`` elements.

    With ``n == block * cores`` this is the single-block-per-core kernel of
    examples/triton-ktir/vector_add_ktir.mlir (same name and arguments)."""
    nblk = n // block
    assert nblk * block == n and nblk % cores == 0
    per_core = nblk // cores
    t = f"tensor<{block}x{dtype}>"
    at = f"!ktdp.access_tile<{block}xindex>"
    body_indent = "    " if per_core == 1 else "      "
    off = "%offset" if per_core == 1 else "%off"
    body = (tile("x_tile", "x_view", [off], [block], [n], dtype, body_indent)
            + tile("y_tile", "y_view", [off], [block], [n], dtype, body_indent)
            + f"{body_indent}%x = ktdp.load %x_tile : {at} -> {t}\n"
            + f"{body_indent}%y = ktdp.load %y_tile : {at} -> {t}\n"
            + f"{body_indent}%output = arith.addf %x, %y : {t}\n"
            + tile("output_tile", "output_view", [off], [block], [n], dtype, body_indent)
            + f"{body_indent}ktdp.store %output, %output_tile : {t}, {at}\n")
    if per_core == 1:
        loop = body
    else:
        loop = (f"    %c0 = arith.constant 0 : index\n"
                f"    %c1 = arith.constant 1 : index\n"
                f"    %nblk = arith.constant {per_core} : index\n"
                f"    scf.for %i = %c0 to %nblk step %c1 {{\n"
                f"      %step = arith.muli %i, %BLOCK_SIZE : index\n"
                f"      %off = arith.addi %offset, %step : index\n"
                + body + "      scf.yield\n    }\n")
    span = "%BLOCK_SIZE" if per_core == 1 else "%span"
    pre = "" if per_core == 1 else (f"    %per_core = arith.constant {per_core} : index\n"
                                    f"    %span = arith.muli %per_core, %BLOCK_SIZE : index\n")
    return (f"module {{\n  func.func @add_kernel(%x_ptr: index, %y_ptr: index, %output_ptr: index, "
            f"%BLOCK_SIZE: index) attributes {{grid = [{cores}, 1]}} {{\n"
            f"    %core_id = ktdp.get_compute_tile_id : index\n" + pre
            + f"    %offset = arith.muli %core_id, {span} : index\n"
            + view("x_view", "x_ptr", [n], dtype) + view("y_view", "y_ptr", [n], dtype)
            + view("output_view", "output_ptr", [n], dtype) + loop + "    return\n  }\n}\n")


# name -> (op text with {x} {y} {t} placeholders, result is a tile of the input dtype)
ELEMENTWISE_OPS = {
    "add": "arith.addf {x}, {y} : {t}", "sub": "arith.subf {x}, {y} : {t}", "mul": "arith.mulf {x}, {y} : {t}",
    "div": "arith.divf {x}, {y} : {t}", "maximum": "arith.maximumf {x}, {y} : {t}",
    "maxnum": "arith.maxnumf {x}, {y} : {t}", "minimum": "arith.minimumf {x}, {y} : {t}",
    "minnum": "arith.minnumf {x}, {y} : {t}", "neg": "arith.negf {x} : {t}", "abs": "math.absf {x} : {t}",
    "sqrt": "math.sqrt {x} : {t}", "exp": "math.exp {x} : {t}", "log": "math.log {x} : {t}",
    "tanh": "math.tanh {x} : {t}", "rsqrt": "math.rsqrt {x} : {t}", "sin": "math.sin {x} : {t}",
    "cos": "math.cos {x} : {t}", "log2": "math.log2 {x} : {t}", "erf": "math.erf {x} : {t}",
}


def elementwise_suite(ops: Sequence[str], n: int = 4096, block: int = 128, cores: int = 4, dtype: str = "f16",
                      select_pred: str = "") -> str:
    """One kernel, one output tensor per entry of ``ops`` (names of ELEMENTWISE_OPS): out_<op> = op(x, y)
    on blocks of ``block`` elements, core c taking blocks c, c + cores, ...  ``select_pred`` (an
    ``arith.cmpf`` predicate such as "olt") adds out_select = select(cmpf pred x y, x, y), and
    ``dtype`` "f16" also adds out_ext_add = truncf(extf x + extf y): the cast ops with an f32 op between."""
    nblk = n // block
    assert nblk * block == n and nblk % cores == 0
    t, at = f"tensor<{block}x{dtype}>", f"!ktdp.access_tile<{block}xindex>"
    names = [f"out_{o}" for o in ops] + (["out_select"] if select_pred else []) + (["out_ext_add"] if dtype == "f16" else [])
    ind = "      "
    body = (tile("x_tile", "x_view", ["%off"], [block], [n], dtype, ind) + tile("y_tile", "y_view", ["%off"], [block], [n], dtype, ind)
            + f"{ind}%x = ktdp.load %x_tile : {at} -> {t}\n{ind}%y = ktdp.load %y_tile : {at} -> {t}\n")
    for o in ops:
        body += f"{ind}%r_{o} = " + ELEMENTWISE_OPS[o].format(x="%x", y="%y", t=t) + "\n"
    if select_pred:
        body += (f"{ind}%keep = arith.cmpf {select_pred}, %x, %y : {t}\n"
                 f"{ind}%r_select = arith.select %keep, %x, %y : tensor<{block}xi1>, {t}\n")
    if dtype == "f16":
        t32 = f"tensor<{block}xf32>"
        body += (f"{ind}%x32 = arith.extf %x : {t} to {t32}\n{ind}%y32 = arith.extf %y : {t} to {t32}\n"
                 f"{ind}%s32 = arith.addf %x32, %y32 : {t32}\n{ind}%r_ext_add = arith.truncf %s32 : {t32} to {t}\n")
    for nm in names:
        body += tile(f"{nm}_tile", f"{nm}_view", ["%off"], [block], [n], dtype, ind)
        body += f"{ind}ktdp.store %r_{nm[4:]}, %{nm}_tile : {t}, {at}\n"
    s = (f"module {{\n  func.func @elementwise_kernel(%x_ptr: index, %y_ptr: index"
         + "".join(f", %{nm}_ptr: index" for nm in names) + f") attributes {{grid = [{cores}, 1]}} {{\n"
         f"    %core_id = ktdp.get_compute_tile_id : index\n"
         f"    %c0 = arith.constant 0 : index\n    %c1 = arith.constant 1 : index\n"
         f"    %blk = arith.constant {block} : index\n    %per_core = arith.constant {nblk // cores} : index\n"
         f"    %ncores = arith.constant {cores} : index\n")
    s += view("x_view", "x_ptr", [n], dtype) + view("y_view", "y_ptr", [n], dtype)
    for nm in names:
        s += view(f"{nm}_view", f"{nm}_ptr", [n], dtype)
    s += (f"    scf.for %i = %c0 to %per_core step %c1 {{\n"
          f"      %b0 = arith.muli %i, %ncores : index\n      %b = arith.addi %b0, %core_id : index\n"
          f"      %off = arith.muli %b, %blk : index\n" + body + "      scf.yield\n    }\n    return\n  }\n}\n")
    return s


def softmax_rows(n_rows: int = 8192, n_cols: int = 4096, cores: int = 32, rows_per_iter: int = 8,
                 f32_stats: bool = True) -> str:
    """Row softmax; core c owns rows [c*R, (c+1)*R), R = n_rows/cores, ``rows_per_iter`` at a time.

    f32_stats: load f16, extend to f32, max/exp/sum/div in f32, truncate to f16
    (the configuration the benchmark is quoted on).  Otherwise all arithmetic
    stays in f16 like examples/triton-ktir/softmax_fwd_ktir.mlir."""
    R = n_rows // cores
    r = rows_per_iter
    assert R * cores == n_rows and R % r == 0
    ct = "f32" if f32_stats else "f16"
    t16, tc, tv = f"tensor<{r}x{n_cols}xf16>", f"tensor<{r}x{n_cols}x{ct}>", f"tensor<{r}x{ct}>"
    at = f"!ktdp.access_tile<{r}x{n_cols}xindex>"
    s = (f"module {{\n  func.func @softmax_kernel(%output_ptr: index, %input_ptr: index) "
         f"attributes {{grid = [{cores}, 1]}} {{\n"
         f"    %core_id = ktdp.get_compute_tile_id : index\n"
         f"    %c0 = arith.constant 0 : index\n"
         f"    %rows = arith.constant {R} : index\n"
         f"    %step = arith.constant {r} : index\n"
         f"    %row0 = arith.muli %core_id, %rows : index\n"
         f"    %row_end = arith.addi %row0, %rows : index\n")
    s += view("input_view", "input_ptr", [n_rows, n_cols], "f16")
    s += view("output_view", "output_ptr", [n_rows, n_cols], "f16")
    s += "    scf.for %row = %row0 to %row_end step %step {\n"
    s += tile("in_tile", "input_view", ["%row", "%c0"], [r, n_cols], [n_rows, n_cols], "f16", "      ")
    s += f"      %x16 = ktdp.load %in_tile : {at} -> {t16}\n"
    if f32_stats:
        s += f"      %x = arith.extf %x16 : {t16} to {tc}\n"
        s += "      %ninf_bits = arith.constant 0xFF800000 : i32\n"
        s += "      %ninf = arith.bitcast %ninf_bits : i32 to f32\n"
        s += "      %zero = arith.constant 0.0 : f32\n"
    else:
        s += "      %ninf = arith.constant 0xFC00 : f16\n"
        s += "      %zero = arith.constant 0.0 : f16\n"
    xin = "%x" if f32_stats else "%x16"
    s += (f"      %max_init = tensor.splat %ninf : {tv}\n"
          f"      %row_max = linalg.reduce {{ arith.maximumf }} ins({xin} : {tc}) outs(%max_init : {tv}) dimensions = [1]\n"
          f"      %bshape = tensor.empty() : {tc}\n"
          f"      %max_b = linalg.broadcast ins(%row_max : {tv}) outs(%bshape : {tc}) dimensions = [1]\n"
          f"      %shifted = arith.subf {xin}, %max_b : {tc}\n"
          f"      %num = math.exp %shifted : {tc}\n"
          f"      %sum_init = tensor.splat %zero : {tv}\n"
          f"      %row_sum = linalg.reduce {{ arith.addf }} ins(%num : {tc}) outs(%sum_init : {tv}) dimensions = [1]\n"
          f"      %sum_b = linalg.broadcast ins(%row_sum : {tv}) outs(%bshape : {tc}) dimensions = [1]\n"
          f"      %y = arith.divf %num, %sum_b : {tc}\n")
    if f32_stats:
        s += f"      %y16 = arith.truncf %y : {tc} to {t16}\n"
    yout = "%y16" if f32_stats else "%y"
    s += tile("out_tile", "output_view", ["%row", "%c0"], [r, n_cols], [n_rows, n_cols], "f16", "      ")
    s += f"      ktdp.store {yout}, %out_tile : {t16}, {at}\n      scf.yield\n    }}\n    return\n  }}\n}}\n"
    return s


def _iat(name: str, vw: str, idx_view: str, base: str, rows: int, cols: int, n_table_rows: int,
         n_idx: int, idx_dtype: str, indent: str) -> str:
    return (f"{indent}%{name} = ktdp.construct_indirect_access_tile\n"
            f"{indent}    intermediate_variables(%d0, %d1)\n"
            f"{indent}    %{vw}[ind(%{idx_view}[{base} + %d0]), (%d1)] {{\n"
            f"{indent}  variables_space_set = {_box([rows, cols])},\n"
            f"{indent}  variables_space_order = {_ident(2)}\n"
            f"{indent}}} : memref<{_xs([n_table_rows, cols], 'f16')}>, memref<{n_idx}x{idx_dtype}>"
            f" -> !ktdp.access_tile<{rows}x{cols}xindex>\n")


def gather_scale_scatter(n_table_rows: int = 65536, cols: int = 128, n_idx: int = 262144,
                         tile_rows: int = 64, cores: int = 64, scale: float = 0.5,
                         idx_dtype: str = "i32") -> str:
    """out[idx] = out[idx] + scale * table[idx], ``tile_rows`` index entries per tile.

    Per tile: gather table rows through the index vector, scale, load the
    destination rows through the same indices, add, scatter back (duplicate
    rows within a tile keep the last writer, tiles apply in order)."""
    per_core = n_idx // cores
    assert per_core * cores == n_idx and per_core % tile_rows == 0
    t = f"tensor<{tile_rows}x{cols}xf16>"
    at = f"!ktdp.access_tile<{tile_rows}x{cols}xindex>"
    s = (f"module {{\n  func.func @gather_scale_scatter(%table_ptr: index, %idx_ptr: index, %out_ptr: index) "
         f"attributes {{grid = [{cores}, 1]}} {{\n"
         f"    %pid = ktdp.get_compute_tile_id : index\n"
         f"    %per_core = arith.constant {per_core} : index\n"
         f"    %tile_rows = arith.constant {tile_rows} : index\n"
         f"    %begin = arith.muli %pid, %per_core : index\n"
         f"    %end = arith.addi %begin, %per_core : index\n"
         f"    %scale = arith.constant {float(scale)} : f16\n")
    s += view("table", "table_ptr", [n_table_rows, cols], "f16")
    s += view("out", "out_ptr", [n_table_rows, cols], "f16")
    s += view("idx", "idx_ptr", [n_idx], idx_dtype)
    s += "    scf.for %base = %begin to %end step %tile_rows {\n"
    s += _iat("src", "table", "idx", "%base", tile_rows, cols, n_table_rows, n_idx, idx_dtype, "      ")
    s += _iat("dst", "out", "idx", "%base", tile_rows, cols, n_table_rows, n_idx, idx_dtype, "      ")
    s += (f"      %rows = ktdp.load %src : {at} -> {t}\n"
          f"      %scale_t = tensor.splat %scale : {t}\n"
          f"      %scaled = arith.mulf %rows, %scale_t : {t}\n"
          f"      %old = ktdp.load %dst : {at} -> {t}\n"
          f"      %new = arith.addf %old, %scaled : {t}\n"
          f"      ktdp.store %new, %dst : {t}, {at}\n"
          f"      scf.yield\n    }}\n    return\n  }}\n}}\n")
    return s


def tiled_matmul(M: int = 4096, N: int = 4096, K: int = 4096, bm: int = 64, bn: int = 64, bk: int = 64,
                 cores: int = 32, f32_acc: bool = True) -> str:
    """C = A @ B with bm x bn output tiles and K-step bk; core c owns tiles [c*T, (c+1)*T).

    f32_acc: operands extended to f32, f32 accumulator carried through the K
    loop, one truncation to f16 at the end.  Otherwise the f16 form of
    examples/triton-ktir/matmul_fwd_ktir.mlir: f16 matmul per K-step added into
    an f16 accumulator."""
    tiles_n = N // bn
    n_tiles = (M // bm) * tiles_n
    per_core = n_tiles // cores
    assert per_core * cores == n_tiles and K % bk == 0
    ct = "f32" if f32_acc else "f16"
    ta, tb = f"tensor<{bm}x{bk}xf16>", f"tensor<{bk}x{bn}xf16>"
    tc16, tcc = f"tensor<{bm}x{bn}xf16>", f"tensor<{bm}x{bn}x{ct}>"
    s = (f"module {{\n  func.func @matmul_kernel(%a_ptr: index, %b_ptr: index, %c_ptr: index) "
         f"attributes {{grid = [{cores}, 1]}} {{\n"
         f"    %pid = ktdp.get_compute_tile_id : index\n"
         f"    %c0 = arith.constant 0 : index\n"
         f"    %c1 = arith.constant 1 : index\n"
         f"    %K = arith.constant {K} : index\n"
         f"    %bm = arith.constant {bm} : index\n"
         f"    %bn = arith.constant {bn} : index\n"
         f"    %bk = arith.constant {bk} : index\n"
         f"    %tiles_n = arith.constant {tiles_n} : index\n"
         f"    %per_core = arith.constant {per_core} : index\n"
         f"    %t_begin = arith.muli %pid, %per_core : index\n"
         f"    %t_end = arith.addi %t_begin, %per_core : index\n")
    s += view("a_view", "a_ptr", [M, K], "f16") + view("b_view", "b_ptr", [K, N], "f16")
    s += view("c_view", "c_ptr", [M, N], "f16")
    s += (f"    scf.for %t = %t_begin to %t_end step %c1 {{\n"
          f"      %tm = arith.divui %t, %tiles_n : index\n"
          f"      %tn = arith.remui %t, %tiles_n : index\n"
          f"      %off_m = arith.muli %tm, %bm : index\n"
          f"      %off_n = arith.muli %tn, %bn : index\n"
          f"      %acc0 = arith.constant dense<0.0> : {tcc}\n"
          f"      %acc = scf.for %off_k = %c0 to %K step %bk iter_args(%acc_it = %acc0) -> ({tcc}) {{\n")
    s += tile("a_tile", "a_view", ["%off_m", "%off_k"], [bm, bk], [M, K], "f16", "        ")
    s += tile("b_tile", "b_view", ["%off_k", "%off_n"], [bk, bn], [K, N], "f16", "        ")
    s += (f"        %a = ktdp.load %a_tile : !ktdp.access_tile<{bm}x{bk}xindex> -> {ta}\n"
          f"        %b = ktdp.load %b_tile : !ktdp.access_tile<{bk}x{bn}xindex> -> {tb}\n")
    if f32_acc:
        s += (f"        %a32 = arith.extf %a : {ta} to tensor<{bm}x{bk}xf32>\n"
              f"        %b32 = arith.extf %b : {tb} to tensor<{bk}x{bn}xf32>\n"
              f"        %next = linalg.matmul ins(%a32, %b32 : tensor<{bm}x{bk}xf32>, tensor<{bk}x{bn}xf32>) "
              f"outs(%acc_it : {tcc}) -> {tcc}\n")
    else:
        s += (f"        %init = tensor.empty() : {tc16}\n"
              f"        %ab = linalg.matmul ins(%a, %b : {ta}, {tb}) outs(%init : {tc16}) -> {tc16}\n"
              f"        %next = arith.addf %acc_it, %ab : {tc16}\n")
    s += f"        scf.yield %next : {tcc}\n      }}\n"
    if f32_acc:
        s += f"      %c16 = arith.truncf %acc : {tcc} to {tc16}\n"
    cval = "%c16" if f32_acc else "%acc"
    s += tile("c_tile", "c_view", ["%off_m", "%off_n"], [bm, bn], [M, N], "f16", "      ")
    s += (f"      ktdp.store {cval}, %c_tile : {tc16}, !ktdp.access_tile<{bm}x{bn}xindex>\n"
          f"      scf.yield\n    }}\n    return\n  }}\n}}\n")
    return s


def blocked_gather(src_shape: Sequence[int], n_selected: Sequence[int], dtype: str = "f16") -> str:
    """out[e0, .., m, n, ..] = src[idx0[e0], .., m, n, ..]: the leading ``len(n_selected)`` dims of
    ``src`` are looked up through index vectors (``idx0``, ``idx1``, ...), the rest taken whole — the
    block gathers of the reference's indirect-load benchmark (expert weights ``X[IDX[e], m, n]``, KV
    pages ``cache[BT[p], h, t, d]``, page/token pairs ``X[P[p], T[t], h]``, expert/head pairs
    ``X[E[e], H[h], m, n]``; benchmarks/bench_utils.py:40-170).  One core loads the whole result as one
    indirect tile and stores it."""
    n_ind = len(n_selected)
    rshape = list(n_selected) + list(src_shape[n_ind:])
    nd = len(src_shape)
    names = [f"%v{i}" for i in range(nd)]
    subs = [f"ind(%idx{i}[{names[i]}])" for i in range(n_ind)] + [f"({names[i]})" for i in range(n_ind, nd)]
    args = ", ".join(["%src_ptr: index"] + [f"%idx{i}_ptr: index" for i in range(n_ind)] + ["%out_ptr: index"])
    t, at = f"tensor<{_xs(rshape, dtype)}>", f"!ktdp.access_tile<{_xs(rshape, 'index')}>"
    s = (f"module {{\n  func.func @blocked_gather({args}) attributes {{grid = [1]}} {{\n"
         f"    %c0 = arith.constant 0 : index\n")
    s += view("src", "src_ptr", list(src_shape), dtype) + view("out", "out_ptr", rshape, dtype)
    for i in range(n_ind):
        s += view(f"idx{i}", f"idx{i}_ptr", [n_selected[i]], "i32")
    idx_types = ", ".join(f"memref<{n_selected[i]}xi32>" for i in range(n_ind))
    s += (f"    %tile = ktdp.construct_indirect_access_tile\n"
          f"        intermediate_variables({', '.join(names)})\n"
          f"        %src[{', '.join(subs)}] {{\n"
          f"      variables_space_set = {_box(rshape)},\n      variables_space_order = {_ident(nd)}\n"
          f"    }} : memref<{_xs(src_shape, dtype)}>, {idx_types} -> {at}\n")
    s += tile("dst", "out", ["%c0"] * nd, rshape, rshape, dtype)
    s += f"    %x = ktdp.load %tile : {at} -> {t}\n    ktdp.store %x, %dst : {t}, {at}\n    return\n  }}\n}}\n"
    return s


def gather_rows_transposed(n_table_rows: int = 32, cols: int = 16, n_idx: int = 64, tile_rows: int = 8,
                           cores: int = 2, idx_dtype: str = "i32") -> str:
    """out[:, e] = table[idx[e], :] — the indirect tile enumerates its (row, column) variable space in
    the order ``variables_space_order = (d0, d1) -> (d1, d0)``, i.e. column by column, so the loaded
    tile is the transpose [cols, tile_rows] of the gathered rows and goes to ``out`` [cols, n_idx] as is."""
    per_core = n_idx // cores
    assert per_core * cores == n_idx and per_core % tile_rows == 0
    t = f"tensor<{cols}x{tile_rows}xf16>"
    s = (f"module {{\n  func.func @gather_rows_transposed(%table_ptr: index, %idx_ptr: index, %out_ptr: index) "
         f"attributes {{grid = [{cores}, 1]}} {{\n"
         f"    %pid = ktdp.get_compute_tile_id : index\n    %c0 = arith.constant 0 : index\n"
         f"    %per_core = arith.constant {per_core} : index\n    %tile_rows = arith.constant {tile_rows} : index\n"
         f"    %begin = arith.muli %pid, %per_core : index\n    %end = arith.addi %begin, %per_core : index\n")
    s += view("table", "table_ptr", [n_table_rows, cols], "f16")
    s += view("out", "out_ptr", [cols, n_idx], "f16")
    s += view("idx", "idx_ptr", [n_idx], idx_dtype)
    s += "    scf.for %base = %begin to %end step %tile_rows {\n"
    s += (f"      %src = ktdp.construct_indirect_access_tile\n"
          f"          intermediate_variables(%d0, %d1)\n"
          f"          %table[ind(%idx[%base + %d0]), (%d1)] {{\n"
          f"        variables_space_set = {_box([tile_rows, cols])},\n"
          f"        variables_space_order = affine_map<(d0, d1) -> (d1, d0)>\n"
          f"      }} : memref<{_xs([n_table_rows, cols], 'f16')}>, memref<{n_idx}x{idx_dtype}>"
          f" -> !ktdp.access_tile<{tile_rows}x{cols}xindex>\n")
    s += tile("dst", "out", ["%c0", "%base"], [cols, tile_rows], [cols, n_idx], "f16", "      ")
    s += (f"      %cols_first = ktdp.load %src : !ktdp.access_tile<{tile_rows}x{cols}xindex> -> {t}\n"
          f"      ktdp.store %cols_first, %dst : {t}, !ktdp.access_tile<{cols}x{tile_rows}xindex>\n"
          f"      scf.yield\n    }}\n    return\n  }}\n}}\n")
    return s


def gather_rows(n_table_rows: int, cols: int, n_idx: int, tile_rows: int, cores: int,
                idx_dtype: str = "i32") -> str:
    """out[e, :] = table[idx[e], :] — indirect load, direct store."""
    per_core = n_idx // cores
    assert per_core * cores == n_idx and per_core % tile_rows == 0
    t = f"tensor<{tile_rows}x{cols}xf16>"
    at = f"!ktdp.access_tile<{tile_rows}x{cols}xindex>"
    s = (f"module {{\n  func.func @gather_rows(%table_ptr: index, %idx_ptr: index, %out_ptr: index) "
         f"attributes {{grid = [{cores}, 1]}} {{\n"
         f"    %pid = ktdp.get_compute_tile_id : index\n"
         f"    %c0 = arith.constant 0 : index\n"
         f"    %per_core = arith.constant {per_core} : index\n"
         f"    %tile_rows = arith.constant {tile_rows} : index\n"
         f"    %begin = arith.muli %pid, %per_core : index\n"
         f"    %end = arith.addi %begin, %per_core : index\n")
    s += view("table", "table_ptr", [n_table_rows, cols], "f16")
    s += view("out", "out_ptr", [n_idx, cols], "f16")
    s += view("idx", "idx_ptr", [n_idx], idx_dtype)
    s += "    scf.for %base = %begin to %end step %tile_rows {\n"
    s += _iat("src", "table", "idx", "%base", tile_rows, cols, n_table_rows, n_idx, idx_dtype, "      ")
    s += tile("dst", "out", ["%base", "%c0"], [tile_rows, cols], [n_idx, cols], "f16", "      ")
    s += (f"      %rows = ktdp.load %src : {at} -> {t}\n"
          f"      ktdp.store %rows, %dst : {t}, {at}\n"
          f"      scf.yield\n    }}\n    return\n  }}\n}}\n")
    return s


def paged_gather(n_seq: int = 4, seq_len: int = 64, page: int = 16, heads: int = 2, dim: int = 32,
                 n_pages: int = 32, chunk: int = 32, dtype: str = "f16") -> str:
    """A paged tensor copied into a dense one: ``out[b, t, h, :] = pages[table[b, t floordiv page], h,
    t mod page, :]`` — the position split into page and slot inside the subscripts of one indirect
    access tile, and the [heads, chunk, dim] tile stored through an access tile that walks the dense
    [seq, heads, dim] layout in the permuted order (h, t, d) -> (t, h, d).  The shape of
    examples/rfc/paged-tensor-copy.mlir of the reference; core b copies sequence b, ``chunk`` positions
    per iteration."""
    assert seq_len % page == 0 and seq_len % chunk == 0
    npg = seq_len // page
    tshape = [heads, chunk, dim]
    t, at = f"tensor<{_xs(tshape, dtype)}>", f"!ktdp.access_tile<{_xs(tshape, 'index')}>"
    s = (f"module {{\n  func.func @paged_gather(%pages_ptr: index, %table_ptr: index, %out_ptr: index) "
         f"attributes {{grid = [{n_seq}]}} {{\n"
         f"    %b = ktdp.get_compute_tile_id : index\n    %c0 = arith.constant 0 : index\n"
         f"    %chunk = arith.constant {chunk} : index\n    %seq_len = arith.constant {seq_len} : index\n")
    s += view("pages", "pages_ptr", [n_pages, heads, page, dim], dtype)
    s += view("table", "table_ptr", [n_seq, npg], "i32")
    s += view("out", "out_ptr", [n_seq, seq_len, heads, dim], dtype)
    s += (f"    scf.for %t0 = %c0 to %seq_len step %chunk {{\n"
          f"      %src = ktdp.construct_indirect_access_tile\n"
          f"          intermediate_variables(%h, %t, %d)\n"
          f"          %pages[ind(%table[%b, (%t0 + %t) floordiv {page}]), (%h), ((%t0 + %t) mod {page}), (%d)] {{\n"
          f"        variables_space_set = {_box(tshape)},\n"
          f"        variables_space_order = {_ident(3)}\n"
          f"      }} : memref<{_xs([n_pages, heads, page, dim], dtype)}>, memref<{_xs([n_seq, npg], 'i32')}>"
          f" -> {at}\n"
          f"      %dst = ktdp.construct_access_tile %out[%b, %t0, %c0, %c0] {{\n"
          f"        access_tile_set = affine_set<(d0, d1, d2, d3) : (d0 >= 0, -d0 >= 0, d1 >= 0, -d1 + {heads - 1} >= 0, "
          f"d2 >= 0, -d2 + {chunk - 1} >= 0, d3 >= 0, -d3 + {dim - 1} >= 0)>,\n"
          f"        access_tile_order = affine_map<(d0, d1, d2, d3) -> (d0, d2, d1, d3)>\n"
          f"      }} : memref<{_xs([n_seq, seq_len, heads, dim], dtype)}> -> !ktdp.access_tile<{_xs([1] + tshape, 'index')}>\n"
          f"      %x = ktdp.load %src : {at} -> {t}\n"
          f"      %x4 = tensor.expand_shape %x [[0, 1], [2], [3]] output_shape [1, {heads}, {chunk}, {dim}] : {t} into "
          f"tensor<{_xs([1] + tshape, dtype)}>\n"
          f"      ktdp.store %x4, %dst : tensor<{_xs([1] + tshape, dtype)}>, !ktdp.access_tile<{_xs([1] + tshape, 'index')}>\n"
          f"      scf.yield\n    }}\n    return\n  }}\n}}\n")
    return s


def scatter_rows(n_out_rows: int, cols: int, n_idx: int, tile_rows: int, cores: int,
                 idx_dtype: str = "i32") -> str:
    """out[idx[e], :] = src[e, :] — direct load, indirect store (last writer of a row wins)."""
    per_core = n_idx // cores
    assert per_core * cores == n_idx and per_core % tile_rows == 0
    t = f"tensor<{tile_rows}x{cols}xf16>"
    at = f"!ktdp.access_tile<{tile_rows}x{cols}xindex>"
    s = (f"module {{\n  func.func @scatter_rows(%src_ptr: index, %idx_ptr: index, %out_ptr: index) "
         f"attributes {{grid = [{cores}, 1]}} {{\n"
         f"    %pid = ktdp.get_compute_tile_id : index\n"
         f"    %c0 = arith.constant 0 : index\n"
         f"    %per_core = arith.constant {per_core} : index\n"
         f"    %tile_rows = arith.constant {tile_rows} : index\n"
         f"    %begin = arith.muli %pid, %per_core : index\n"
         f"    %end = arith.addi %begin, %per_core : index\n")
    s += view("src", "src_ptr", [n_idx, cols], "f16")
    s += view("out", "out_ptr", [n_out_rows, cols], "f16")
    s += view("idx", "idx_ptr", [n_idx], idx_dtype)
    s += "    scf.for %base = %begin to %end step %tile_rows {\n"
    s += tile("from", "src", ["%base", "%c0"], [tile_rows, cols], [n_idx, cols], "f16", "      ")
    s += _iat("to", "out", "idx", "%base", tile_rows, cols, n_out_rows, n_idx, idx_dtype, "      ")
    s += (f"      %rows = ktdp.load %from : {at} -> {t}\n"
          f"      ktdp.store %rows, %to : {t}, {at}\n"
          f"      scf.yield\n    }}\n    return\n  }}\n}}\n")
    return s


def causal_attention(seq: int = 2048, heads: int = 256, head_dim: int = 128, tile_m: int = 128,
                     tile_n: int = 128) -> str:
    """Blockwise causal attention with online softmax in f32 and paged K/V.

    Query / output are [seq, heads, head_dim] f16 (batch folded into heads); the
    K and V caches are [seq/tile_n, tile_n, heads, head_dim] f16 pages reached
    through a block table (an identity table gives dense attention).  Core
    (q, h) owns query rows [q*tile_m, (q+1)*tile_m) of head h and walks
    ``num_tiles`` KV pages carrying (running max M, running sum L, accumulator).
    Same computation as examples/triton-ktir/paged_attention.mlir of the
    reference with one query head per KV head: M starts at -inf, L at 1.0,
    masked scores are -inf, the epilogue divides by L and truncates to f16."""
    assert seq % tile_m == 0 and seq % tile_n == 0
    nb = seq // tile_n
    tm, tn, hd, H = tile_m, tile_n, head_dim, heads
    qv, cv = [seq, H, hd], [nb, tn, H, hd]
    f = lambda shp, dt: f"tensor<{_xs(shp, dt)}>"   # noqa: E731

    def kv_tile(name, vw):
        return (f"      %{name} = ktdp.construct_indirect_access_tile\n"
                f"          intermediate_variables(%d0, %d1, %d2, %d3)\n"
                f"          %{vw}[ind(%block_tables[%c0, %j + %d0]), (%d1), (%pid_h + %d2), (%d3)] {{\n"
                f"        variables_space_set = {_box([1, tn, 1, hd])},\n"
                f"        variables_space_order = {_ident(4)}\n"
                f"      }} : memref<{_xs(cv, 'f16')}>, memref<1x{nb}xi32> -> !ktdp.access_tile<{_xs([1, tn, 1, hd], 'index')}>\n")

    s = (f"module {{\n  func.func @attention_kernel(%output_ptr: index, %query_ptr: index, %key_cache_ptr: index,\n"
         f"      %value_cache_ptr: index, %block_tables_ptr: index, %num_tiles: index, %context_len: index,\n"
         f"      %scale: f32) attributes {{grid = [{seq // tm}, {H}]}} {{\n"
         f"    %pid_q, %pid_h = ktdp.get_compute_tile_id : index, index\n"
         f"    %c0 = arith.constant 0 : index\n"
         f"    %c1 = arith.constant 1 : index\n"
         f"    %c_tm = arith.constant {tm} : index\n"
         f"    %c_tn = arith.constant {tn} : index\n"
         f"    %ninf_bits = arith.constant 0xFF800000 : i32\n"
         f"    %ninf = arith.bitcast %ninf_bits : i32 to f32\n"
         f"    %zero = arith.constant 0.0 : f32\n"
         f"    %one = arith.constant 1.0 : f32\n"
         f"    %q_row0 = arith.muli %pid_q, %c_tm : index\n"
         f"    %q_abs0 = arith.addi %q_row0, %context_len : index\n")
    s += view("query", "query_ptr", qv, "f16") + view("output", "output_ptr", qv, "f16")
    s += view("key_cache", "key_cache_ptr", cv, "f16") + view("value_cache", "value_cache_ptr", cv, "f16")
    s += view("block_tables", "block_tables_ptr", [1, nb], "i32")
    s += tile("q_tile", "query", ["%q_row0", "%pid_h", "%c0"], [tm, 1, hd], qv, "f16")
    s += (f"    %q3 = ktdp.load %q_tile : !ktdp.access_tile<{_xs([tm, 1, hd], 'index')}> -> {f([tm, 1, hd], 'f16')}\n"
          f"    %q16 = tensor.collapse_shape %q3 [[0, 1], [2]] : {f([tm, 1, hd], 'f16')} into {f([tm, hd], 'f16')}\n"
          f"    %q = arith.extf %q16 : {f([tm, hd], 'f16')} to {f([tm, hd], 'f32')}\n"
          f"    %m_init = tensor.splat %ninf : {f([tm], 'f32')}\n"
          f"    %l_init = tensor.splat %one : {f([tm], 'f32')}\n"
          f"    %acc_init = tensor.splat %zero : {f([tm, hd], 'f32')}\n"
          f"    %m_fin, %l_fin, %acc_fin = scf.for %j = %c0 to %num_tiles step %c1\n"
          f"        iter_args(%m_run = %m_init, %l_run = %l_init, %acc = %acc_init)\n"
          f"        -> ({f([tm], 'f32')}, {f([tm], 'f32')}, {f([tm, hd], 'f32')}) {{\n")
    s += kv_tile("k_tile", "key_cache") + kv_tile("v_tile", "value_cache")
    t4, t2 = f([1, tn, 1, hd], "f16"), f([tn, hd], "f16")
    at4 = f"!ktdp.access_tile<{_xs([1, tn, 1, hd], 'index')}>"
    s += (f"      %k4 = ktdp.load %k_tile : {at4} -> {t4}\n"
          f"      %v4 = ktdp.load %v_tile : {at4} -> {t4}\n"
          f"      %k2 = tensor.collapse_shape %k4 [[0, 1], [2, 3]] : {t4} into {t2}\n"
          f"      %v2 = tensor.collapse_shape %v4 [[0, 1], [2, 3]] : {t4} into {t2}\n"
          f"      %kt_init = tensor.empty() : {f([hd, tn], 'f16')}\n"
          f"      %kt16 = linalg.transpose ins(%k2 : {t2}) outs(%kt_init : {f([hd, tn], 'f16')}) permutation = [1, 0]\n"
          f"      %kt = arith.extf %kt16 : {f([hd, tn], 'f16')} to {f([hd, tn], 'f32')}\n"
          f"      %v = arith.extf %v2 : {t2} to {f([tn, hd], 'f32')}\n"
          f"      %s_zero = tensor.splat %zero : {f([tm, tn], 'f32')}\n"
          f"      %qk = linalg.matmul ins(%q, %kt : {f([tm, hd], 'f32')}, {f([hd, tn], 'f32')}) "
          f"outs(%s_zero : {f([tm, tn], 'f32')}) -> {f([tm, tn], 'f32')}\n"
          f"      %scale_t = tensor.splat %scale : {f([tm, tn], 'f32')}\n"
          f"      %sc = arith.mulf %scale_t, %qk : {f([tm, tn], 'f32')}\n"
          f"      %col0 = arith.muli %j, %c_tn : index\n"
          f"      %masked_init = tensor.empty() : {f([tm, tn], 'f32')}\n"
          f"      %masked = linalg.generic {{\n"
          f"          indexing_maps = [{_ident(2)}, {_ident(2)}],\n"
          f"          iterator_types = [\"parallel\", \"parallel\"]}}\n"
          f"          ins(%sc : {f([tm, tn], 'f32')}) outs(%masked_init : {f([tm, tn], 'f32')}) {{\n"
          f"        ^bb0(%s_val : f32, %unused : f32):\n"
          f"          %r = linalg.index 0 : index\n"
          f"          %c = linalg.index 1 : index\n"
          f"          %q_pos = arith.addi %q_abs0, %r : index\n"
          f"          %k_pos = arith.addi %col0, %c : index\n"
          f"          %keep = arith.cmpi ule, %k_pos, %q_pos : index\n"
          f"          %sel = arith.select %keep, %s_val, %ninf : f32\n"
          f"          linalg.yield %sel : f32\n"
          f"      }} -> {f([tm, tn], 'f32')}\n"
          f"      %rmax_init = tensor.splat %ninf : {f([tm], 'f32')}\n"
          f"      %rmax = linalg.reduce {{ arith.maximumf }} ins(%masked : {f([tm, tn], 'f32')}) "
          f"outs(%rmax_init : {f([tm], 'f32')}) dimensions = [1]\n"
          f"      %m_new = arith.maximumf %m_run, %rmax : {f([tm], 'f32')}\n"
          f"      %bs = tensor.empty() : {f([tm, tn], 'f32')}\n"
          f"      %m_b = linalg.broadcast ins(%m_new : {f([tm], 'f32')}) outs(%bs : {f([tm, tn], 'f32')}) dimensions = [1]\n"
          f"      %shift = arith.subf %masked, %m_b : {f([tm, tn], 'f32')}\n"
          f"      %p = math.exp %shift : {f([tm, tn], 'f32')}\n"
          f"      %lsum_init = tensor.splat %zero : {f([tm], 'f32')}\n"
          f"      %lsum = linalg.reduce {{ arith.addf }} ins(%p : {f([tm, tn], 'f32')}) "
          f"outs(%lsum_init : {f([tm], 'f32')}) dimensions = [1]\n"
          f"      %dm = arith.subf %m_run, %m_new : {f([tm], 'f32')}\n"
          f"      %alpha = math.exp %dm : {f([tm], 'f32')}\n"
          f"      %bo = tensor.empty() : {f([tm, hd], 'f32')}\n"
          f"      %alpha_b = linalg.broadcast ins(%alpha : {f([tm], 'f32')}) outs(%bo : {f([tm, hd], 'f32')}) dimensions = [1]\n"
          f"      %acc_scaled = arith.mulf %acc, %alpha_b : {f([tm, hd], 'f32')}\n"
          f"      %acc_new = linalg.matmul ins(%p, %v : {f([tm, tn], 'f32')}, {f([tn, hd], 'f32')}) "
          f"outs(%acc_scaled : {f([tm, hd], 'f32')}) -> {f([tm, hd], 'f32')}\n"
          f"      %l_scaled = arith.mulf %l_run, %alpha : {f([tm], 'f32')}\n"
          f"      %l_new = arith.addf %l_scaled, %lsum : {f([tm], 'f32')}\n"
          f"      scf.yield %m_new, %l_new, %acc_new : {f([tm], 'f32')}, {f([tm], 'f32')}, {f([tm, hd], 'f32')}\n"
          f"    }}\n"
          f"    %bo2 = tensor.empty() : {f([tm, hd], 'f32')}\n"
          f"    %l_b = linalg.broadcast ins(%l_fin : {f([tm], 'f32')}) outs(%bo2 : {f([tm, hd], 'f32')}) dimensions = [1]\n"
          f"    %o32 = arith.divf %acc_fin, %l_b : {f([tm, hd], 'f32')}\n"
          f"    %o16 = arith.truncf %o32 : {f([tm, hd], 'f32')} to {f([tm, hd], 'f16')}\n"
          f"    %o3 = tensor.expand_shape %o16 [[0, 1], [2]] output_shape [{tm}, 1, {hd}] : "
          f"{f([tm, hd], 'f16')} into {f([tm, 1, hd], 'f16')}\n")
    s += tile("o_tile", "output", ["%q_row0", "%pid_h", "%c0"], [tm, 1, hd], qv, "f16")
    s += (f"    ktdp.store %o3, %o_tile : {f([tm, 1, hd], 'f16')}, !ktdp.access_tile<{_xs([tm, 1, hd], 'index')}>\n"
          f"    return\n  }}\n}}\n")
    return s


def _generic(res: str, ins, out_shape, body_args, body, indent="      ") -> str:
    """``linalg.generic`` over parallel dims: ``ins`` = [(ssa name, shape)], a row vector broadcasts
    along the last dim of ``out_shape``; ``body`` = lines of the region ending in the yielded name."""
    nd = len(out_shape)
    dims = ", ".join(f"d{i}" for i in range(nd))
    maps = [f"affine_map<({dims}) -> ({', '.join(f'd{i}' for i in range(len(shp)))})>" for _, shp in ins]
    maps.append(_ident(nd))
    f = lambda shp: f"tensor<{_xs(shp, 'f32')}>"   # noqa: E731
    lines = [f"{indent}%{res}_out = tensor.empty() : {f(out_shape)}",
             f"{indent}%{res} = linalg.generic {{",
             f"{indent}    indexing_maps = [{', '.join(maps)}],",
             f"{indent}    iterator_types = [{', '.join(['\"parallel\"'] * nd)}]}}",
             f"{indent}    ins({', '.join('%' + n for n, _ in ins)} : {', '.join(f(shp) for _, shp in ins)})",
             f"{indent}    outs(%{res}_out : {f(out_shape)}) {{",
             f"{indent}  ^bb0({', '.join(f'%{a} : f32' for a in body_args)}, %{res}_o : f32):"]
    lines += [f"{indent}    {ln}" for ln in body[:-1]]
    lines += [f"{indent}    linalg.yield %{body[-1]} : f32", f"{indent}}} -> {f(out_shape)}"]
    return "\n".join(lines) + "\n"


def paged_attention(num_tokens: int = 2048, context_len: int = 2048, num_query_heads: int = 256,
                    num_kv_heads: int = 256, head_dim: int = 128, block_size: int = 128, block_q: int = 128) -> str:
    """Paged attention with online softmax, the kernel shape of the reference's own generator
    (notebooks/demo_gen_mlir.py:724-1012; examples/triton-ktir/paged_attention.mlir:163-433): same
    function name, arguments and op sequence, so either text drives the same device kernel.

    Grid = [num_tokens / block_q, num_kv_heads].  A core owns ``block_q`` query positions of the
    ``num_query_heads / num_kv_heads`` query heads that share its K/V head: its tile is
    [block_q, group, head_dim], collapsed position-major to [block_q * group, head_dim].  Per KV page
    (``block_size`` rows, reached through the block table): S = scale * Q K^T, masked to
    kv position <= context_len + query position (row / group inside a ``linalg.generic``),
    m = max(M, rowmax S), P = exp(S - m), alpha = exp(M - m), acc = acc * alpha + P V,
    L = L * alpha + rowsum P with M = -inf, L = 1.0 to start; O = acc / L as f16.  With an identity
    block table, ``context_len = 0`` and ``num_tiles = num_tokens / block_size`` this is dense causal
    attention over [num_tokens, heads, head_dim] (a batch folds into the heads)."""
    grp = num_query_heads // num_kv_heads
    bq, bs, hd, nt = block_q, block_size, head_dim, num_tokens
    bm = grp * bq
    nb = (context_len + bs - 1) // bs
    qv, cv = [nt, num_query_heads, hd], [nb, bs, num_kv_heads, hd]
    f = lambda shp, dt="f32": f"tensor<{_xs(shp, dt)}>"   # noqa: E731
    q3, at3 = [bq, grp, hd], f"!ktdp.access_tile<{_xs([bq, grp, hd], 'index')}>"

    def kv_tile(name, vw):
        return (f"      %{name} = ktdp.construct_indirect_access_tile\n"
                f"          intermediate_variables(%d0, %d1, %d2, %d3)\n"
                f"          %{vw}[ind(%block_tables[%c0, %bt_idx + %d0]), (%d1), (%pid1 + %d2), (%d3)] {{\n"
                f"        variables_space_set = {_box([1, bs, 1, hd])},\n"
                f"        variables_space_order = {_ident(4)}\n"
                f"      }} : memref<{_xs(cv, 'f16')}>, memref<1x{nb}xi32> -> !ktdp.access_tile<{_xs([1, bs, 1, hd], 'index')}>\n")

    s = (f"module {{\n  func.func @paged_attention_kernel(%output_ptr: index, %query_ptr: index, %key_cache_ptr: index,\n"
         f"      %value_cache_ptr: index, %block_tables_ptr: index, %cur_batch_start_index: index,\n"
         f"      %block_table_offset: index, %num_tiles: index, %context_len: index, %scale: f32)\n"
         f"      attributes {{grid = [{nt // bq}, {num_kv_heads}]}} {{\n"
         f"    %pid0, %pid1 = ktdp.get_compute_tile_id : index, index\n"
         f"    %c0 = arith.constant 0 : index\n"
         f"    %c1 = arith.constant 1 : index\n"
         f"    %c_bq = arith.constant {bq} : index\n"
         f"    %c_grp = arith.constant {grp} : index\n"
         f"    %c_bs = arith.constant {bs} : index\n"
         f"    %q_rel0 = arith.muli %pid0, %c_bq : index\n"
         f"    %q_row0 = arith.addi %cur_batch_start_index, %q_rel0 : index\n"
         f"    %q_head0 = arith.muli %pid1, %c_grp : index\n"
         f"    %ninf_bits = arith.constant 0xFF800000 : i32\n"
         f"    %ninf = arith.bitcast %ninf_bits : i32 to f32\n"
         f"    %zero = arith.constant 0.0 : f32\n"
         f"    %one = arith.constant 1.0 : f32\n")
    s += view("query", "query_ptr", qv, "f16") + view("output", "output_ptr", qv, "f16")
    s += view("key_cache", "key_cache_ptr", cv, "f16") + view("value_cache", "value_cache_ptr", cv, "f16")
    s += view("block_tables", "block_tables_ptr", [1, nb], "i32")
    s += tile("q_tile", "query", ["%q_row0", "%q_head0", "%c0"], q3, qv, "f16")
    s += (f"    %q3 = ktdp.load %q_tile : {at3} -> {f(q3, 'f16')}\n"
          f"    %q16 = tensor.collapse_shape %q3 [[0, 1], [2]] : {f(q3, 'f16')} into {f([bm, hd], 'f16')}\n"
          f"    %q = arith.extf %q16 : {f([bm, hd], 'f16')} to {f([bm, hd])}\n"
          f"    %m_init = tensor.splat %ninf : {f([bm])}\n"
          f"    %l_init = tensor.splat %one : {f([bm])}\n"
          f"    %acc_init = tensor.splat %zero : {f([bm, hd])}\n"
          f"    %m_fin, %l_fin, %acc_fin = scf.for %j = %c0 to %num_tiles step %c1\n"
          f"        iter_args(%m_run = %m_init, %l_run = %l_init, %acc = %acc_init)\n"
          f"        -> ({f([bm])}, {f([bm])}, {f([bm, hd])}) {{\n"
          f"      %bt_idx = arith.addi %block_table_offset, %j : index\n")
    s += kv_tile("k_tile", "key_cache") + kv_tile("v_tile", "value_cache")
    t4, t2 = f([1, bs, 1, hd], "f16"), f([bs, hd], "f16")
    at4 = f"!ktdp.access_tile<{_xs([1, bs, 1, hd], 'index')}>"
    s += (f"      %k4 = ktdp.load %k_tile : {at4} -> {t4}\n"
          f"      %v4 = ktdp.load %v_tile : {at4} -> {t4}\n"
          f"      %k2 = tensor.collapse_shape %k4 [[0, 1], [2, 3]] : {t4} into {t2}\n"
          f"      %v2 = tensor.collapse_shape %v4 [[0, 1], [2, 3]] : {t4} into {t2}\n"
          f"      %kt_init = tensor.empty() : {f([hd, bs], 'f16')}\n"
          f"      %kt16 = linalg.transpose ins(%k2 : {t2}) outs(%kt_init : {f([hd, bs], 'f16')}) permutation = [1, 0]\n"
          f"      %kt = arith.extf %kt16 : {f([hd, bs], 'f16')} to {f([hd, bs])}\n"
          f"      %v = arith.extf %v2 : {t2} to {f([bs, hd])}\n"
          f"      %s_zero = tensor.splat %zero : {f([bm, bs])}\n"
          f"      %qk = linalg.matmul ins(%q, %kt : {f([bm, hd])}, {f([hd, bs])}) "
          f"outs(%s_zero : {f([bm, bs])}) -> {f([bm, bs])}\n"
          f"      %scale_t = tensor.splat %scale : {f([bm, bs])}\n"
          f"      %sc = arith.mulf %scale_t, %qk : {f([bm, bs])}\n")
    s += _generic("masked", [("sc", [bm, bs])], [bm, bs], ["s_val"], [
        "%r = linalg.index 0 : index",
        "%c = linalg.index 1 : index",
        "%q_in_tile = arith.divui %r, %c_grp : index",
        "%q_rel = arith.addi %q_rel0, %q_in_tile : index",
        "%q_pos = arith.addi %context_len, %q_rel : index",
        "%col0 = arith.muli %j, %c_bs : index",
        "%k_pos = arith.addi %col0, %c : index",
        "%keep = arith.cmpi ule, %k_pos, %q_pos : index",
        "%sel = arith.select %keep, %s_val, %ninf : f32",
        "sel"])
    s += (f"      %rmax_init = tensor.splat %ninf : {f([bm])}\n"
          f"      %rmax = linalg.reduce ins(%masked : {f([bm, bs])}) outs(%rmax_init : {f([bm])}) dimensions = [1]\n"
          f"          (%ra : f32, %rb : f32) {{\n"
          f"        %rm = arith.maximumf %ra, %rb : f32\n"
          f"        linalg.yield %rm : f32\n"
          f"      }}\n")
    s += _generic("m_new", [("m_run", [bm]), ("rmax", [bm])], [bm], ["mo", "mn"],
                  ["%mm = arith.maximumf %mo, %mn : f32", "mm"])
    s += _generic("p", [("masked", [bm, bs]), ("m_new", [bm])], [bm, bs], ["sv", "mv"],
                  ["%sh = arith.subf %sv, %mv : f32", "%ex = math.exp %sh : f32", "ex"])
    s += (f"      %lsum_init = tensor.splat %zero : {f([bm])}\n"
          f"      %lsum = linalg.reduce ins(%p : {f([bm, bs])}) outs(%lsum_init : {f([bm])}) dimensions = [1]\n"
          f"          (%sa : f32, %sb : f32) {{\n"
          f"        %ss = arith.addf %sa, %sb : f32\n"
          f"        linalg.yield %ss : f32\n"
          f"      }}\n")
    s += _generic("alpha", [("m_run", [bm]), ("m_new", [bm])], [bm], ["mo", "mn"],
                  ["%dm = arith.subf %mo, %mn : f32", "%ea = math.exp %dm : f32", "ea"])
    s += _generic("acc_scaled", [("acc", [bm, hd]), ("alpha", [bm])], [bm, hd], ["av", "al"],
                  ["%sa2 = arith.mulf %av, %al : f32", "sa2"])
    s += (f"      %acc_new = linalg.matmul ins(%p, %v : {f([bm, bs])}, {f([bs, hd])}) "
          f"outs(%acc_scaled : {f([bm, hd])}) -> {f([bm, hd])}\n")
    s += _generic("l_new", [("l_run", [bm]), ("alpha", [bm]), ("lsum", [bm])], [bm], ["lv", "al", "lj"],
                  ["%la = arith.mulf %lv, %al : f32", "%ln = arith.addf %la, %lj : f32", "ln"])
    s += (f"      scf.yield %m_new, %l_new, %acc_new : {f([bm])}, {f([bm])}, {f([bm, hd])}\n"
          f"    }}\n")
    s += _generic("o32", [("acc_fin", [bm, hd]), ("l_fin", [bm])], [bm, hd], ["av", "lv"],
                  ["%dv = arith.divf %av, %lv : f32", "dv"], indent="    ")
    s += (f"    %o16 = arith.truncf %o32 : {f([bm, hd])} to {f([bm, hd], 'f16')}\n"
          f"    %o3 = tensor.expand_shape %o16 [[0, 1], [2]] output_shape [{bq}, {grp}, {hd}] : "
          f"{f([bm, hd], 'f16')} into {f(q3, 'f16')}\n")
    s += tile("o_tile", "output", ["%q_row0", "%q_head0", "%c0"], q3, qv, "f16")
    s += (f"    ktdp.store %o3, %o_tile : {f(q3, 'f16')}, {at3}\n"
          f"    return\n  }}\n}}\n")
    return s


def ring_allreduce(n_cores: int = 4, group: int = 4, cols: int = 128, combine: str = "add", dtype: str = "f16",
                   inner: int = 1, strided: bool = False, absent_core: int = -1) -> str:
    """Cross-core all-reduce inside groups of ``group`` cores (the op pair of examples/ktir/ring_reduce.mlir
    and examples/latency/ring_reduce_multi_group.mlir of the reference): core c loads row c of ``in``
    ([n_cores * inner, cols]), the cores of a group combine their rows through
    ``ktdp.inter_tile_produce`` / ``ktdp.inter_tile_reduce`` (``combine``: add, mul, max), and EVERY core
    stores what it holds to row c of ``out`` — each core folds in ring arrival order, so rows of one
    group may differ in the last bit.  ``inner`` > 1 repeats this for ``inner`` rows per core in a
    loop; ``strided`` makes group g the cores {g, g + n_groups, ...} instead of a contiguous range.
    ``absent_core`` >= 0 puts the whole exchange under a condition that this core does not take: its
    ring neighbours then wait for ever, which the interpreter must report as a deadlock."""
    assert n_cores % group == 0 and (absent_core < 0 or inner == 1)
    ng = n_cores // group
    t, at = f"tensor<1x{cols}x{dtype}>", f"!ktdp.access_tile<1x{cols}xindex>"
    rows = n_cores * inner
    if strided:
        members = f"affine_set<(i)[g] : (i - g >= 0, (i - g) mod {ng} == 0, -i + {n_cores - 1} >= 0)>"
    else:
        members = f"affine_set<(i)[g] : (i - {group} * g >= 0, -i + {group} * g + {group - 1} >= 0)>"
    groups = f"affine_set<(g) : (g >= 0, -g + {ng - 1} >= 0)>"
    body_op = {"add": f"linalg.add ins(%lhs, %rhs : {t}, {t}) outs(%init : {t}) -> {t}",
               "max": f"linalg.max ins(%lhs, %rhs : {t}, {t}) outs(%init : {t}) -> {t}",
               "mul": f"arith.mulf %lhs, %rhs : {t}"}[combine]
    ident = {"add": "0.0", "max": "-65504.0", "mul": "1.0"}[combine]
    ind = "      " if inner > 1 else "    "
    body = (tile("in_tile", "in_view", ["%row", "%c0"], [1, cols], [rows, cols], dtype, ind)
            + f"{ind}%partial = ktdp.load %in_tile : {at} -> {t}\n"
            + f"{ind}%fut = ktdp.inter_tile_produce\n{ind}    producer_tiles_per_group = #ring_members\n"
              f"{ind}    : {t} -> !ktdp.tile_future<{t}, groups = {groups}>\n{ind}{{\n"
              f"{ind}  ^bb0(%gid: index):\n{ind}    ktdp.yield_partial %partial : {t}\n{ind}}}\n"
            + f"{ind}%id_init = tensor.empty() : {t}\n"
              f"{ind}%ident = linalg.fill ins(%c_ident : {dtype}) outs(%id_init : {t}) -> {t}\n"
            + f"{ind}%reduced = ktdp.inter_tile_reduce(%fut)\n{ind}    consumer_tiles_per_group = #ring_members,\n"
              f"{ind}    identity(%ident : {t}) : !ktdp.tile_future<{t}, groups = {groups}> -> {t}\n{ind}{{\n"
              f"{ind}  ^bb0(%lhs: {t}, %rhs: {t}):\n{ind}    %init = tensor.empty() : {t}\n"
              f"{ind}    %comb = {body_op}\n{ind}    ktdp.yield_reduced %comb : {t}\n{ind}}}\n"
            + tile("out_tile", "out_view", ["%row", "%c0"], [1, cols], [rows, cols], dtype, ind)
            + f"{ind}ktdp.store %reduced, %out_tile : {t}, {at}\n")
    s = (f"#ring_members = {members}\n\n"
         f"module {{\n  func.func @ring_allreduce(%in_ptr: index, %out_ptr: index) attributes {{grid = [{n_cores}]}} {{\n"
         f"    %pid = ktdp.get_compute_tile_id : index\n    %c0 = arith.constant 0 : index\n"
         f"    %c1 = arith.constant 1 : index\n    %c_inner = arith.constant {inner} : index\n"
         f"    %c_ident = arith.constant {ident} : {dtype}\n"
         f"    %row0 = arith.muli %pid, %c_inner : index\n")
    s += view("in_view", "in_ptr", [rows, cols], dtype) + view("out_view", "out_ptr", [rows, cols], dtype)
    if inner > 1:
        s += (f"    scf.for %i = %c0 to %c_inner step %c1 {{\n      %row = arith.addi %row0, %i : index\n"
              + body + "      scf.yield\n    }\n")
    elif absent_core >= 0:
        s += (f"    %row = arith.addi %row0, %c0 : index\n    %c_absent = arith.constant {absent_core} : index\n"
              f"    %present = arith.cmpi ne, %pid, %c_absent : index\n    scf.if %present {{\n"
              + body.replace("\n    ", "\n      ").replace("    %in_tile", "      %in_tile", 1) + "    }\n")
    else:
        s += "    %row = arith.addi %row0, %c0 : index\n" + body
    return s + "    return\n  }\n}\n"


def shared_slot_store(n_cores: int = 4, slots: int = 2, cols: int = 64, dtype: str = "f16") -> str:
    """Every core doubles its row of ``x`` ([n_cores, cols]) and stores it to row ``core % slots`` of
    ``out`` ([slots, cols]): several cores write the same bytes, and the reference — which runs its
    cores one after the other (ktir_cpu/grid.py:595-613) — keeps the value of the highest core id."""
    t, at = f"tensor<1x{cols}x{dtype}>", f"!ktdp.access_tile<1x{cols}xindex>"
    return (f"module {{\n  func.func @shared_slot(%x_ptr: index, %out_ptr: index) attributes {{grid = [{n_cores}, 1]}} {{\n"
            f"    %c = ktdp.get_compute_tile_id : index\n    %c0 = arith.constant 0 : index\n"
            f"    %n_slots = arith.constant {slots} : index\n    %slot = arith.remui %c, %n_slots : index\n"
            + view("x_view", "x_ptr", [n_cores, cols], dtype) + view("out_view", "out_ptr", [slots, cols], dtype)
            + tile("x_tile", "x_view", ["%c", "%c0"], [1, cols], [n_cores, cols], dtype)
            + tile("out_tile", "out_view", ["%slot", "%c0"], [1, cols], [slots, cols], dtype)
            + f"    %x = ktdp.load %x_tile : {at} -> {t}\n    %twice = arith.addf %x, %x : {t}\n"
              f"    ktdp.store %twice, %out_tile : {t}, {at}\n    return\n  }}\n}}\n")


def _box_at(lo: Sequence[int], hi: Sequence[int]) -> str:
    """affine_set of the box [lo, hi) (hi exclusive)."""
    dims = ", ".join(f"d{i}" for i in range(len(lo)))
    cons = ", ".join(f"d{i} - {l} >= 0, -d{i} + {h - 1} >= 0" for i, (l, h) in enumerate(zip(lo, hi)))
    return f"affine_set<({dims}) : ({cons})>"


def _part(name: str, ptr: str, lo, hi, strides, dtype: str) -> str:
    shape = [h - l for l, h in zip(lo, hi)]
    return (f"    %{name} = ktdp.construct_memory_view %{ptr}, sizes: {shape}, strides: {list(strides)} {{\n"
            f"      coordinate_set = {_box_at(lo, hi)}, memory_space = #ktdp.memory_space<global>\n"
            f"    }} : memref<{_xs(shape, dtype)}>\n")


def _dist(name: str, parts, shapes, shape, dtype: str) -> str:
    names = ", ".join(f"%{p_}" for p_ in parts)
    types = ", ".join(f"memref<{_xs(s_, dtype)}>" for s_ in shapes)
    return (f"    %{name} = ktdp.construct_distributed_memory_view\n"
            f"        ({names} : {types})\n        : memref<{_xs(shape, dtype)}>\n")


def sharded_scale(rows: int = 64, cols: int = 64, tile_rows: int = 8, cores: int = 4, shift: int = 0,
                  dtype: str = "f16") -> str:
    """out = a + a on a [rows, cols] tensor that lives in three pieces — rows [0, rows/2) row-major in
    ``a0``, rows [rows/2, rows) x cols [0, cols/2) COLUMN-major in ``a1``, the remaining quarter
    row-major in ``a2`` — read through one distributed memory view, and written through another one
    that splits the columns between ``o0`` and ``o1``.  Core c handles ``rows / cores / tile_rows``
    tiles of ``tile_rows`` full rows starting at row ``c * rows / cores + shift``: with a shift that is
    not a multiple of the tile height a tile crosses the row boundary between the partitions, every
    tile crosses the column boundaries, and the last tile hangs over the end of the tensor (what no
    partition backs reads as zero and is not written)."""
    h, w = rows // 2, cols // 2
    per_core = rows // cores
    n_iter = per_core // tile_rows
    assert h * 2 == rows and w * 2 == cols and n_iter * tile_rows * cores == rows and 0 <= shift < tile_rows
    t, at = f"tensor<{_xs([tile_rows, cols], dtype)}>", f"!ktdp.access_tile<{_xs([tile_rows, cols], 'index')}>"
    s = (f"module {{\n  func.func @sharded_scale(%a0_ptr: index, %a1_ptr: index, %a2_ptr: index, %o0_ptr: index, "
         f"%o1_ptr: index) attributes {{grid = [{cores}, 1]}} {{\n"
         f"    %core = ktdp.get_compute_tile_id : index\n"
         f"    %c0 = arith.constant 0 : index\n    %c1 = arith.constant 1 : index\n"
         f"    %n_iter = arith.constant {n_iter} : index\n    %th = arith.constant {tile_rows} : index\n"
         f"    %per_core = arith.constant {per_core} : index\n    %shift = arith.constant {shift} : index\n"
         f"    %row_lo = arith.muli %core, %per_core : index\n    %row0 = arith.addi %row_lo, %shift : index\n")
    s += _part("a0", "a0_ptr", [0, 0], [h, cols], [cols, 1], dtype)
    s += _part("a1", "a1_ptr", [h, 0], [rows, w], [1, h], dtype)
    s += _part("a2", "a2_ptr", [h, w], [rows, cols], [w, 1], dtype)
    s += _dist("a_all", ["a0", "a1", "a2"], [[h, cols], [h, w], [h, w]], [rows, cols], dtype)
    s += _part("o0", "o0_ptr", [0, 0], [rows, w], [w, 1], dtype)
    s += _part("o1", "o1_ptr", [0, w], [rows, cols], [w, 1], dtype)
    s += _dist("o_all", ["o0", "o1"], [[rows, w], [rows, w]], [rows, cols], dtype)
    s += (f"    scf.for %i = %c0 to %n_iter step %c1 {{\n"
          f"      %step = arith.muli %i, %th : index\n      %r = arith.addi %row0, %step : index\n"
          + tile("a_tile", "a_all", ["%r", "%c0"], [tile_rows, cols], [rows, cols], dtype, "      ")
          + f"      %x = ktdp.load %a_tile : {at} -> {t}\n      %y = arith.addf %x, %x : {t}\n"
          + tile("o_tile", "o_all", ["%r", "%c0"], [tile_rows, cols], [rows, cols], dtype, "      ")
          + f"      ktdp.store %y, %o_tile : {t}, {at}\n      scf.yield\n    }}\n    return\n  }}\n}}\n")
    return s


def sharded_center(cols: int = 256, cores: int = 4, rows: int = 8, dtype: str = "f16") -> str:
    """Tensor-parallel row centering: y = x - sum_over_all_columns(x) / cols.  x and y are [rows, cols];
    core c owns the column block c of both, declared as partition c of a distributed memory view
    (all partitions inside the one tensor).  Per row: local sum over the core's columns, all-reduce of
    the [1, 1] partial sums over the cores (ring), subtract.  Every access tile lies whole inside one
    partition, so the loads and stores are ordinary strided tiles on the device; the shape of
    examples/latency/rmsnorm_4core_2x2.mlir of the reference."""
    w = cols // cores
    assert w * cores == cols
    t, at = f"tensor<1x{w}x{dtype}>", f"!ktdp.access_tile<1x{w}xindex>"
    tv = f"tensor<1x1x{dtype}>"
    groups = "affine_set<(g) : (g >= 0, -g >= 0)>"
    s = (f"#all_cores = affine_set<(i)[g] : (i >= 0, -i + {cores - 1} >= 0)>\n\n"
         f"module {{\n  func.func @sharded_center(%x_ptr: index, %y_ptr: index) attributes {{grid = [{cores}]}} {{\n"
         f"    %core = ktdp.get_compute_tile_id : index\n    %c0 = arith.constant 0 : index\n"
         f"    %c1 = arith.constant 1 : index\n    %rows = arith.constant {rows} : index\n"
         f"    %w = arith.constant {w} : index\n    %col0 = arith.muli %core, %w : index\n"
         f"    %zero = arith.constant 0.0 : {dtype}\n    %inv_n = arith.constant {1.0 / cols} : {dtype}\n")
    for nm, ptr in (("x", "x_ptr"), ("y", "y_ptr")):
        names = []
        for c in range(cores):
            s += (f"    %{nm}_off{c} = arith.constant {c * w} : index\n"
                  f"    %{nm}_base{c} = arith.addi %{ptr}, %{nm}_off{c} : index\n")
            s += _part(f"{nm}_p{c}", f"{nm}_base{c}", [0, c * w], [rows, (c + 1) * w], [cols, 1], dtype)
            names.append(f"{nm}_p{c}")
        s += _dist(f"{nm}_all", names, [[rows, w]] * cores, [rows, cols], dtype)
    ind = "      "
    s += f"    scf.for %row = %c0 to %rows step %c1 {{\n"
    s += tile("x_tile", "x_all", ["%row", "%col0"], [1, w], [rows, cols], dtype, ind)
    s += (f"{ind}%x = ktdp.load %x_tile : {at} -> {t}\n"
          f"{ind}%acc0 = tensor.splat %zero : tensor<1x{dtype}>\n"
          f"{ind}%sum = linalg.reduce {{ arith.addf }} ins(%x : {t}) outs(%acc0 : tensor<1x{dtype}>) dimensions = [1]\n"
          f"{ind}%partial = tensor.expand_shape %sum [[0, 1]] output_shape [1, 1] : tensor<1x{dtype}> into {tv}\n"
          f"{ind}%fut = ktdp.inter_tile_produce\n{ind}    producer_tiles_per_group = #all_cores\n"
          f"{ind}    : {tv} -> !ktdp.tile_future<{tv}, groups = {groups}>\n{ind}{{\n"
          f"{ind}  ^bb0(%gid: index):\n{ind}    ktdp.yield_partial %partial : {tv}\n{ind}}}\n"
          f"{ind}%ident = tensor.splat %zero : {tv}\n"
          f"{ind}%total = ktdp.inter_tile_reduce(%fut)\n{ind}    consumer_tiles_per_group = #all_cores,\n"
          f"{ind}    identity(%ident : {tv}) : !ktdp.tile_future<{tv}, groups = {groups}> -> {tv}\n{ind}{{\n"
          f"{ind}  ^bb0(%lhs: {tv}, %rhs: {tv}):\n{ind}    %comb = arith.addf %lhs, %rhs : {tv}\n"
          f"{ind}    ktdp.yield_reduced %comb : {tv}\n{ind}}}\n"
          f"{ind}%inv_n_t = tensor.splat %inv_n : {tv}\n"
          f"{ind}%mean = arith.mulf %total, %inv_n_t : {tv}\n"
          f"{ind}%bshape = tensor.empty() : {t}\n"
          f"{ind}%mean_row = tensor.collapse_shape %mean [[0, 1]] : {tv} into tensor<1x{dtype}>\n"
          f"{ind}%mean_b = linalg.broadcast ins(%mean_row : tensor<1x{dtype}>) outs(%bshape : {t}) dimensions = [1]\n"
          f"{ind}%y = arith.subf %x, %mean_b : {t}\n")
    s += tile("y_tile", "y_all", ["%row", "%col0"], [1, w], [rows, cols], dtype, ind)
    s += f"{ind}ktdp.store %y, %y_tile : {t}, {at}\n{ind}scf.yield\n    }}\n    return\n  }}\n}}\n"
    return s


def region_reduce_rows(n_rows: int = 16, n_cols: int = 37, cores: int = 4, dtype: str = "f16") -> str:
    """Two row reductions whose combiners are regions of several ops: ``mx[r] = max over the row``
    written as ``arith.cmpf ogt`` + ``arith.select`` (examples/ktir/reduce_multiop.mlir of the
    reference), and ``sa[r]``, the fold of ``(in, out) -> |in - out| * 0.5 + in`` — neither symmetric nor
    associative, so its value pins the order of the pairwise fold (left half with right half, odd slice
    carried, the folded value as lhs of the final combine with the initial value).
    ``n_cols`` may be odd at any level."""
    R = n_rows // cores
    assert R * cores == n_rows
    t, at = f"tensor<1x{n_cols}x{dtype}>", f"!ktdp.access_tile<1x{n_cols}xindex>"
    tv, atv = f"tensor<1x{dtype}>", "!ktdp.access_tile<1xindex>"
    s = (f"module {{\n  func.func @region_reduce(%x_ptr: index, %mx_ptr: index, %sa_ptr: index) "
         f"attributes {{grid = [{cores}, 1]}} {{\n"
         f"    %core_id = ktdp.get_compute_tile_id : index\n"
         f"    %c0 = arith.constant 0 : index\n    %c1 = arith.constant 1 : index\n"
         f"    %rows = arith.constant {R} : index\n    %row0 = arith.muli %core_id, %rows : index\n"
         f"    %row_end = arith.addi %row0, %rows : index\n"
         f"    %ninf = arith.constant 0xFC00 : {dtype}\n    %zero = arith.constant 0.0 : {dtype}\n"
         f"    %half_c = arith.constant 0.5 : {dtype}\n")
    s += view("x_view", "x_ptr", [n_rows, n_cols], dtype)
    s += view("mx_view", "mx_ptr", [n_rows], dtype) + view("sa_view", "sa_ptr", [n_rows], dtype)
    s += f"    scf.for %row = %row0 to %row_end step %c1 {{\n"
    s += tile("x_tile", "x_view", ["%row", "%c0"], [1, n_cols], [n_rows, n_cols], dtype, "      ")
    s += (f"      %x = ktdp.load %x_tile : {at} -> {t}\n"
          f"      %mx_init = tensor.splat %ninf : {tv}\n"
          f"      %mx = linalg.reduce ins(%x : {t}) outs(%mx_init : {tv}) dimensions = [1]\n"
          f"        (%in: {dtype}, %out: {dtype}) {{\n"
          f"          %gt = arith.cmpf ogt, %in, %out : {dtype}\n"
          f"          %sel = arith.select %gt, %in, %out : {dtype}\n"
          f"          linalg.yield %sel : {dtype}\n        }}\n"
          f"      %sa_init = tensor.splat %zero : {tv}\n"
          f"      %sa = linalg.reduce ins(%x : {t}) outs(%sa_init : {tv}) dimensions = [1]\n"
          f"        (%in2: {dtype}, %out2: {dtype}) {{\n"
          f"          %df = arith.subf %in2, %out2 : {dtype}\n"
          f"          %ab = math.absf %df : {dtype}\n"
          f"          %hf = arith.mulf %ab, %half_c : {dtype}\n"
          f"          %sm = arith.addf %hf, %in2 : {dtype}\n"
          f"          linalg.yield %sm : {dtype}\n        }}\n")
    s += tile("mx_tile", "mx_view", ["%row"], [1], [n_rows], dtype, "      ")
    s += tile("sa_tile", "sa_view", ["%row"], [1], [n_rows], dtype, "      ")
    s += (f"      ktdp.store %mx, %mx_tile : {tv}, {atv}\n      ktdp.store %sa, %sa_tile : {tv}, {atv}\n"
          f"      scf.yield\n    }}\n    return\n  }}\n}}\n")
    return s


def generic_contraction(M: int = 8, N: int = 16, K: int = 24, cores: int = 2, dtype: str = "f32") -> str:
    """C = A @ B + C0 written as one ``linalg.generic`` with a reduction iterator (maps (m, n, k) ->
    (m, k), (k, n), (m, n); body mulf + addf into the outs argument) — the contraction form of the
    reference's ``linalg.generic`` tests (tests/test_dialects_exec.py:1218-1283).  Core c computes
    ``M / cores`` rows; the products over k are folded pairwise, not summed in k order."""
    R = M // cores
    assert R * cores == M
    ta, tb, tc = f"tensor<{R}x{K}x{dtype}>", f"tensor<{K}x{N}x{dtype}>", f"tensor<{R}x{N}x{dtype}>"
    s = (f"module {{\n  func.func @generic_contraction(%a_ptr: index, %b_ptr: index, %c_ptr: index) "
         f"attributes {{grid = [{cores}, 1]}} {{\n"
         f"    %core_id = ktdp.get_compute_tile_id : index\n    %c0 = arith.constant 0 : index\n"
         f"    %rows = arith.constant {R} : index\n    %row0 = arith.muli %core_id, %rows : index\n")
    s += view("a_view", "a_ptr", [M, K], dtype) + view("b_view", "b_ptr", [K, N], dtype) + view("c_view", "c_ptr", [M, N], dtype)
    s += tile("a_tile", "a_view", ["%row0", "%c0"], [R, K], [M, K], dtype)
    s += tile("b_tile", "b_view", ["%c0", "%c0"], [K, N], [K, N], dtype)
    s += tile("c_tile", "c_view", ["%row0", "%c0"], [R, N], [M, N], dtype)
    s += (f"    %a = ktdp.load %a_tile : !ktdp.access_tile<{R}x{K}xindex> -> {ta}\n"
          f"    %b = ktdp.load %b_tile : !ktdp.access_tile<{K}x{N}xindex> -> {tb}\n"
          f"    %c_init = ktdp.load %c_tile : !ktdp.access_tile<{R}x{N}xindex> -> {tc}\n"
          f"    %c = linalg.generic {{\n"
          f"        indexing_maps = [affine_map<(d0, d1, d2) -> (d0, d2)>, affine_map<(d0, d1, d2) -> (d2, d1)>, "
          f"affine_map<(d0, d1, d2) -> (d0, d1)>],\n"
          f"        iterator_types = [\"parallel\", \"parallel\", \"reduction\"]}}\n"
          f"        ins(%a, %b : {ta}, {tb})\n        outs(%c_init : {tc}) {{\n"
          f"      ^bb0(%aa : {dtype}, %bb : {dtype}, %cc : {dtype}):\n"
          f"        %prod = arith.mulf %aa, %bb : {dtype}\n"
          f"        %acc = arith.addf %prod, %cc : {dtype}\n"
          f"        linalg.yield %acc : {dtype}\n    }} -> {tc}\n"
          f"    ktdp.store %c, %c_tile : {tc}, !ktdp.access_tile<{R}x{N}xindex>\n    return\n  }}\n}}\n")
    return s


def layernorm_rows(n_rows: int = 64, n_cols: int = 256, cores: int = 4, eps: float = 1e-5) -> str:
    """y = (x - mean) / sqrt(var + eps) * w + b per row, f32 statistics, one row per iteration.

    The op mix of examples/triton-ktir/layernorm_fwd_ktir.mlir (sum reduction, broadcast, rsqrt,
    per-column weight and bias) at a size of one's choosing; also writes the row means."""
    R = n_rows // cores
    assert R * cores == n_rows
    t16, t32, tv = f"tensor<1x{n_cols}xf16>", f"tensor<1x{n_cols}xf32>", "tensor<1xf32>"
    at, atv = f"!ktdp.access_tile<1x{n_cols}xindex>", "!ktdp.access_tile<1xindex>"
    s = (f"module {{\n  func.func @layernorm_kernel(%x_ptr: index, %w_ptr: index, %b_ptr: index, %y_ptr: index, "
         f"%mean_ptr: index) attributes {{grid = [{cores}, 1]}} {{\n"
         f"    %core_id = ktdp.get_compute_tile_id : index\n"
         f"    %c0 = arith.constant 0 : index\n    %c1 = arith.constant 1 : index\n"
         f"    %rows = arith.constant {R} : index\n"
         f"    %row0 = arith.muli %core_id, %rows : index\n"
         f"    %row_end = arith.addi %row0, %rows : index\n"
         f"    %zero = arith.constant 0.0 : f32\n"
         f"    %inv_n = arith.constant {1.0 / n_cols} : f32\n"
         f"    %eps = arith.constant {eps} : f32\n")
    s += view("x_view", "x_ptr", [n_rows, n_cols], "f16") + view("y_view", "y_ptr", [n_rows, n_cols], "f16")
    s += view("w_view", "w_ptr", [1, n_cols], "f16") + view("b_view", "b_ptr", [1, n_cols], "f16")
    s += view("mean_view", "mean_ptr", [n_rows], "f32")
    s += tile("w_tile", "w_view", ["%c0", "%c0"], [1, n_cols], [1, n_cols], "f16")
    s += tile("b_tile", "b_view", ["%c0", "%c0"], [1, n_cols], [1, n_cols], "f16")
    s += (f"    %w16 = ktdp.load %w_tile : {at} -> {t16}\n    %b16 = ktdp.load %b_tile : {at} -> {t16}\n"
          f"    %w = arith.extf %w16 : {t16} to {t32}\n    %b = arith.extf %b16 : {t16} to {t32}\n"
          f"    scf.for %row = %row0 to %row_end step %c1 {{\n")
    s += tile("x_tile", "x_view", ["%row", "%c0"], [1, n_cols], [n_rows, n_cols], "f16", "      ")
    s += (f"      %x16 = ktdp.load %x_tile : {at} -> {t16}\n"
          f"      %x = arith.extf %x16 : {t16} to {t32}\n"
          f"      %acc0 = tensor.splat %zero : {tv}\n"
          f"      %sum = linalg.reduce {{ arith.addf }} ins(%x : {t32}) outs(%acc0 : {tv}) dimensions = [1]\n"
          f"      %inv_n_t = tensor.splat %inv_n : {tv}\n"
          f"      %mean = arith.mulf %sum, %inv_n_t : {tv}\n"
          f"      %bshape = tensor.empty() : {t32}\n"
          f"      %mean_b = linalg.broadcast ins(%mean : {tv}) outs(%bshape : {t32}) dimensions = [1]\n"
          f"      %xc = arith.subf %x, %mean_b : {t32}\n"
          f"      %sq = arith.mulf %xc, %xc : {t32}\n"
          f"      %acc1 = tensor.splat %zero : {tv}\n"
          f"      %ssq = linalg.reduce {{ arith.addf }} ins(%sq : {t32}) outs(%acc1 : {tv}) dimensions = [1]\n"
          f"      %var = arith.mulf %ssq, %inv_n_t : {tv}\n"
          f"      %eps_t = tensor.splat %eps : {tv}\n"
          f"      %var_eps = arith.addf %var, %eps_t : {tv}\n"
          f"      %rstd = math.rsqrt %var_eps : {tv}\n"
          f"      %rstd_b = linalg.broadcast ins(%rstd : {tv}) outs(%bshape : {t32}) dimensions = [1]\n"
          f"      %xn = arith.mulf %xc, %rstd_b : {t32}\n"
          f"      %xw = arith.mulf %xn, %w : {t32}\n"
          f"      %y = arith.addf %xw, %b : {t32}\n"
          f"      %y16 = arith.truncf %y : {t32} to {t16}\n")
    s += tile("y_tile", "y_view", ["%row", "%c0"], [1, n_cols], [n_rows, n_cols], "f16", "      ")
    s += tile("m_tile", "mean_view", ["%row"], [1], [n_rows], "f32", "      ")
    s += (f"      ktdp.store %y16, %y_tile : {t16}, {at}\n"
          f"      ktdp.store %mean, %m_tile : {tv}, {atv}\n"
          f"      scf.yield\n    }}\n    return\n  }}\n}}\n")
    return s


def naive_attention(seq: int = 64, head_dim: int = 32, cores: int = 2) -> str:
    """softmax(Q K^T * scale) V with whole-tile matmuls, a transpose and f32 softmax — the shape of
    examples/triton-ktir/sdpa_2d.mlir: each core handles a block of query rows against all of K and V."""
    R = seq // cores
    assert R * cores == seq
    tq, tk = f"tensor<{R}x{head_dim}xf16>", f"tensor<{seq}x{head_dim}xf16>"
    tq32, tk32, tkt = f"tensor<{R}x{head_dim}xf32>", f"tensor<{seq}x{head_dim}xf32>", f"tensor<{head_dim}x{seq}xf32>"
    ts, tv = f"tensor<{R}x{seq}xf32>", f"tensor<{R}xf32>"
    atq, atk = f"!ktdp.access_tile<{R}x{head_dim}xindex>", f"!ktdp.access_tile<{seq}x{head_dim}xindex>"
    s = (f"module {{\n  func.func @naive_attention(%q_ptr: index, %k_ptr: index, %v_ptr: index, %o_ptr: index) "
         f"attributes {{grid = [{cores}, 1]}} {{\n"
         f"    %core_id = ktdp.get_compute_tile_id : index\n"
         f"    %c0 = arith.constant 0 : index\n"
         f"    %rows = arith.constant {R} : index\n"
         f"    %row0 = arith.muli %core_id, %rows : index\n"
         f"    %scale = arith.constant {head_dim ** -0.5} : f32\n"
         f"    %zero = arith.constant 0.0 : f32\n"
         f"    %ninf_bits = arith.constant 0xFF800000 : i32\n"
         f"    %ninf = arith.bitcast %ninf_bits : i32 to f32\n")
    for nm in ("q", "k", "v", "o"):
        s += view(f"{nm}_view", f"{nm}_ptr", [seq, head_dim], "f16")
    s += tile("q_tile", "q_view", ["%row0", "%c0"], [R, head_dim], [seq, head_dim], "f16")
    s += tile("k_tile", "k_view", ["%c0", "%c0"], [seq, head_dim], [seq, head_dim], "f16")
    s += tile("v_tile", "v_view", ["%c0", "%c0"], [seq, head_dim], [seq, head_dim], "f16")
    s += tile("o_tile", "o_view", ["%row0", "%c0"], [R, head_dim], [seq, head_dim], "f16")
    s += (f"    %q16 = ktdp.load %q_tile : {atq} -> {tq}\n"
          f"    %k16 = ktdp.load %k_tile : {atk} -> {tk}\n"
          f"    %v16 = ktdp.load %v_tile : {atk} -> {tk}\n"
          f"    %q = arith.extf %q16 : {tq} to {tq32}\n"
          f"    %k = arith.extf %k16 : {tk} to {tk32}\n"
          f"    %v = arith.extf %v16 : {tk} to {tk32}\n"
          f"    %kt_init = tensor.empty() : {tkt}\n"
          f"    %kt = linalg.transpose ins(%k : {tk32}) outs(%kt_init : {tkt}) permutation = [1, 0]\n"
          f"    %s_init = tensor.splat %zero : {ts}\n"
          f"    %s = linalg.matmul ins(%q, %kt : {tq32}, {tkt}) outs(%s_init : {ts}) -> {ts}\n"
          f"    %scale_t = tensor.splat %scale : {ts}\n"
          f"    %ss = arith.mulf %s, %scale_t : {ts}\n"
          f"    %m_init = tensor.splat %ninf : {tv}\n"
          f"    %m = linalg.reduce {{ arith.maximumf }} ins(%ss : {ts}) outs(%m_init : {tv}) dimensions = [1]\n"
          f"    %bshape = tensor.empty() : {ts}\n"
          f"    %m_b = linalg.broadcast ins(%m : {tv}) outs(%bshape : {ts}) dimensions = [1]\n"
          f"    %sh = arith.subf %ss, %m_b : {ts}\n"
          f"    %p = math.exp %sh : {ts}\n"
          f"    %l_init = tensor.splat %zero : {tv}\n"
          f"    %l = linalg.reduce {{ arith.addf }} ins(%p : {ts}) outs(%l_init : {tv}) dimensions = [1]\n"
          f"    %l_b = linalg.broadcast ins(%l : {tv}) outs(%bshape : {ts}) dimensions = [1]\n"
          f"    %pn = arith.divf %p, %l_b : {ts}\n"
          f"    %o_init = tensor.splat %zero : {tq32}\n"
          f"    %o = linalg.matmul ins(%pn, %v : {ts}, {tk32}) outs(%o_init : {tq32}) -> {tq32}\n"
          f"    %o16 = arith.truncf %o : {tq32} to {tq}\n"
          f"    ktdp.store %o16, %o_tile : {tq}, {atq}\n"
          f"    return\n  }}\n}}\n")
    return s


def gather_elements(n_rows: int = 32, n_cols: int = 16, n_src: int = 64) -> str:
    """out[i, j] = src[idx[i, j], j] — an indirect access tile whose index varies along both tile
    dimensions (the general form of examples/rfc/indirect-access-copy.mlir), one core."""
    t = f"tensor<{n_rows}x{n_cols}xf16>"
    at = f"!ktdp.access_tile<{n_rows}x{n_cols}xindex>"
    s = (f"module {{\n  func.func @gather_elements(%src_ptr: index, %idx_ptr: index, %out_ptr: index) "
         f"attributes {{grid = [1, 1]}} {{\n    %c0 = arith.constant 0 : index\n")
    s += view("src", "src_ptr", [n_src, n_cols], "f16") + view("idx", "idx_ptr", [n_rows, n_cols], "i32")
    s += view("out", "out_ptr", [n_rows, n_cols], "f16")
    s += (f"    %g = ktdp.construct_indirect_access_tile\n"
          f"        intermediate_variables(%d0, %d1)\n"
          f"        %src[ind(%idx[%d0, %d1]), (%d1)] {{\n"
          f"      variables_space_set = {_box([n_rows, n_cols])},\n"
          f"      variables_space_order = {_ident(2)}\n"
          f"    }} : memref<{_xs([n_src, n_cols], 'f16')}>, memref<{_xs([n_rows, n_cols], 'i32')}>"
          f" -> {at}\n")
    s += tile("o_tile", "out", ["%c0", "%c0"], [n_rows, n_cols], [n_rows, n_cols], "f16")
    s += (f"    %vals = ktdp.load %g : {at} -> {t}\n"
          f"    ktdp.store %vals, %o_tile : {t}, {at}\n    return\n  }}\n}}\n")
    return s


def update_in_place(n_rows: int = 64, cols: int = 64, tile_rows: int = 8, cores: int = 2, loop: bool = True,
                    reuse_new: bool = False) -> str:
    """x = 2 * x in place, old = the x from before: each tile is loaded ONCE, its double stored back
    over it, and the loaded tile stored to ``old`` afterwards — so ``old`` holds the values from
    before the first store although its own store comes second.  ``loop``: the tiles of a core in an
    ``scf.for`` (both stores inside it), else one tile per core.  ``reuse_new``: ``old`` instead gets
    ``loaded tile + tile loaded again after the first store`` (= 3 * x), which ties the second store
    to memory both before and after the first."""
    per_core = n_rows // cores
    assert per_core * cores == n_rows and per_core % tile_rows == 0 and (loop or per_core == tile_rows)
    t, at = f"tensor<{tile_rows}x{cols}xf16>", f"!ktdp.access_tile<{tile_rows}x{cols}xindex>"
    s = (f"module {{\n  func.func @update_in_place(%x_ptr: index, %old_ptr: index) attributes {{grid = [{cores}, 1]}} {{\n"
         f"    %pid = ktdp.get_compute_tile_id : index\n    %c0 = arith.constant 0 : index\n"
         f"    %per_core = arith.constant {per_core} : index\n    %tile_rows = arith.constant {tile_rows} : index\n"
         f"    %begin = arith.muli %pid, %per_core : index\n    %end = arith.addi %begin, %per_core : index\n")
    s += view("x", "x_ptr", [n_rows, cols], "f16") + view("old", "old_ptr", [n_rows, cols], "f16")
    ind = "      " if loop else "    "
    row = "%r" if loop else "%begin"
    if loop:
        s += "    scf.for %r = %begin to %end step %tile_rows {\n"
    s += tile("xt", "x", [row, "%c0"], [tile_rows, cols], [n_rows, cols], "f16", ind)
    s += tile("ot", "old", [row, "%c0"], [tile_rows, cols], [n_rows, cols], "f16", ind)
    s += (f"{ind}%a = ktdp.load %xt : {at} -> {t}\n{ind}%b = arith.addf %a, %a : {t}\n"
          f"{ind}ktdp.store %b, %xt : {t}, {at}\n")
    if reuse_new:
        s += f"{ind}%n = ktdp.load %xt : {at} -> {t}\n{ind}%s = arith.addf %a, %n : {t}\n{ind}ktdp.store %s, %ot : {t}, {at}\n"
    else:
        s += f"{ind}ktdp.store %a, %ot : {t}, {at}\n"
    if loop:
        s += "      scf.yield\n    }\n"
    return s + "    return\n  }\n}\n"


def shifted_reuse(n_rows: int = 64, cols: int = 64, tile_rows: int = 8) -> str:
    """One core, one ``scf.for`` over row tiles: tile ``i`` of ``b`` gets ``2 * a[i]``, then tile ``i``
    of ``c`` gets tile ``i + 1`` of ``b`` — which the loop has not written yet, so ``c`` holds what
    ``b`` held on entry (the last tile reads row tile 0 again, already doubled)."""
    t, at = f"tensor<{tile_rows}x{cols}xf16>", f"!ktdp.access_tile<{tile_rows}x{cols}xindex>"
    s = (f"module {{\n  func.func @shifted_reuse(%a_ptr: index, %b_ptr: index, %c_ptr: index) attributes {{grid = [1, 1]}} {{\n"
         f"    %c0 = arith.constant 0 : index\n    %n = arith.constant {n_rows} : index\n"
         f"    %tile_rows = arith.constant {tile_rows} : index\n")
    for nm in "abc":
        s += view(nm, f"{nm}_ptr", [n_rows, cols], "f16")
    s += ("    scf.for %r = %c0 to %n step %tile_rows {\n"
          "      %r1 = arith.addi %r, %tile_rows : index\n      %nx = arith.remui %r1, %n : index\n")
    s += tile("at", "a", ["%r", "%c0"], [tile_rows, cols], [n_rows, cols], "f16", "      ")
    s += tile("bt", "b", ["%r", "%c0"], [tile_rows, cols], [n_rows, cols], "f16", "      ")
    s += tile("bn", "b", ["%nx", "%c0"], [tile_rows, cols], [n_rows, cols], "f16", "      ")
    s += tile("ct", "c", ["%r", "%c0"], [tile_rows, cols], [n_rows, cols], "f16", "      ")
    s += (f"      %x = ktdp.load %at : {at} -> {t}\n      %y = arith.addf %x, %x : {t}\n"
          f"      ktdp.store %y, %bt : {t}, {at}\n      %z = ktdp.load %bn : {at} -> {t}\n"
          f"      ktdp.store %z, %ct : {t}, {at}\n      scf.yield\n    }}\n    return\n  }}\n}}\n")
    return s


def core_chain(n_cores: int = 8, cols: int = 64, dtype: str = "f16") -> str:
    """x[c + 1] += x[c] on core c: every core reads the row the core before it has just written, so
    the core-after-core order of the reference turns the rows into running sums (row r ends as
    x[0] + ... + x[r], rounded to the tile dtype at every step)."""
    t, at = f"tensor<1x{cols}x{dtype}>", f"!ktdp.access_tile<1x{cols}xindex>"
    rows = n_cores + 1
    s = (f"module {{\n  func.func @core_chain(%x_ptr: index) attributes {{grid = [{n_cores}, 1]}} {{\n"
         f"    %c = ktdp.get_compute_tile_id : index\n    %c0 = arith.constant 0 : index\n"
         f"    %c1 = arith.constant 1 : index\n    %n = arith.addi %c, %c1 : index\n")
    s += view("x", "x_ptr", [rows, cols], dtype)
    s += tile("prev", "x", ["%c", "%c0"], [1, cols], [rows, cols], dtype)
    s += tile("mine", "x", ["%n", "%c0"], [1, cols], [rows, cols], dtype)
    s += (f"    %a = ktdp.load %prev : {at} -> {t}\n    %b = ktdp.load %mine : {at} -> {t}\n"
          f"    %s = arith.addf %a, %b : {t}\n    ktdp.store %s, %mine : {t}, {at}\n    return\n  }}\n}}\n")
    return s


def accumulate_rows(n_cores: int = 4, per_core: int = 6, cols: int = 64, dtype: str = "f16") -> str:
    """acc[c] += x[c * per_core + i] for i = 0 .. per_core - 1, the running row re-loaded from memory
    and stored back in every iteration of an ``scf.for`` — each iteration reads what the one before it
    wrote (rounded to the tile dtype), so the iterations only make sense one after the other."""
    t, at = f"tensor<1x{cols}x{dtype}>", f"!ktdp.access_tile<1x{cols}xindex>"
    rows = n_cores * per_core
    s = (f"module {{\n  func.func @accumulate_rows(%x_ptr: index, %acc_ptr: index) attributes {{grid = [{n_cores}, 1]}} {{\n"
         f"    %c = ktdp.get_compute_tile_id : index\n    %c0 = arith.constant 0 : index\n"
         f"    %c1 = arith.constant 1 : index\n    %per_core = arith.constant {per_core} : index\n"
         f"    %begin = arith.muli %c, %per_core : index\n    %end = arith.addi %begin, %per_core : index\n")
    s += view("x", "x_ptr", [rows, cols], dtype) + view("acc", "acc_ptr", [n_cores, cols], dtype)
    s += tile("at", "acc", ["%c", "%c0"], [1, cols], [n_cores, cols], dtype)
    s += "    scf.for %r = %begin to %end step %c1 {\n"
    s += tile("xt", "x", ["%r", "%c0"], [1, cols], [rows, cols], dtype, "      ")
    s += (f"      %a = ktdp.load %at : {at} -> {t}\n      %b = ktdp.load %xt : {at} -> {t}\n"
          f"      %s = arith.addf %a, %b : {t}\n      ktdp.store %s, %at : {t}, {at}\n      scf.yield\n    }}\n"
          f"    return\n  }}\n}}\n")
    return s


def rmsnorm_rows(n_rows: int = 64, n_cols: int = 256, cores: int = 4, tile_rows: int = 4, eps: float = 1e-6,
                 weight: bool = False) -> str:
    """y = x / sqrt(mean(x^2) + eps) per row, ``tile_rows`` rows per iteration, f32 statistics; also writes
    the per-row 1 / sqrt(mean(x^2) + eps) — one reduction, one per-row value broadcast back, a stored
    tile with one value per row.  ``weight``: y is also multiplied by a weight row ``w[n_cols]`` that is
    loaded once and broadcast over the rows of every tile (``%w_ptr`` becomes the second argument)."""
    R = n_rows // cores
    assert R * cores == n_rows and R % tile_rows == 0
    t16, t32, tv = f"tensor<{tile_rows}x{n_cols}xf16>", f"tensor<{tile_rows}x{n_cols}xf32>", f"tensor<{tile_rows}xf32>"
    at, atv = f"!ktdp.access_tile<{tile_rows}x{n_cols}xindex>", f"!ktdp.access_tile<{tile_rows}xindex>"
    wv = f"tensor<{n_cols}xf16>", f"tensor<{n_cols}xf32>", f"!ktdp.access_tile<{n_cols}xindex>"
    s = (f"module {{\n  func.func @rmsnorm_kernel(%x_ptr: index, {'%w_ptr: index, ' if weight else ''}%y_ptr: index, %rstd_ptr: index) "
         f"attributes {{grid = [{cores}, 1]}} {{\n"
         f"    %core_id = ktdp.get_compute_tile_id : index\n"
         f"    %c0 = arith.constant 0 : index\n    %step = arith.constant {tile_rows} : index\n"
         f"    %rows = arith.constant {R} : index\n"
         f"    %row0 = arith.muli %core_id, %rows : index\n"
         f"    %row_end = arith.addi %row0, %rows : index\n"
         f"    %zero = arith.constant 0.0 : f32\n"
         f"    %inv_n = arith.constant {1.0 / n_cols} : f32\n"
         f"    %eps = arith.constant {eps} : f32\n")
    s += view("x_view", "x_ptr", [n_rows, n_cols], "f16") + view("y_view", "y_ptr", [n_rows, n_cols], "f16")
    s += view("rstd_view", "rstd_ptr", [n_rows], "f32")
    if weight:
        s += view("w_view", "w_ptr", [n_cols], "f16") + tile("w_tile", "w_view", ["%c0"], [n_cols], [n_cols], "f16")
    s += "    scf.for %row = %row0 to %row_end step %step {\n"
    if weight:
        s += (f"      %w16 = ktdp.load %w_tile : {wv[2]} -> {wv[0]}\n      %w1 = arith.extf %w16 : {wv[0]} to {wv[1]}\n"
              f"      %wshape = tensor.empty() : {t32}\n"
              f"      %w = linalg.broadcast ins(%w1 : {wv[1]}) outs(%wshape : {t32}) dimensions = [0]\n")
    s += tile("x_tile", "x_view", ["%row", "%c0"], [tile_rows, n_cols], [n_rows, n_cols], "f16", "      ")
    s += (f"      %x16 = ktdp.load %x_tile : {at} -> {t16}\n"
          f"      %x = arith.extf %x16 : {t16} to {t32}\n"
          f"      %sq = arith.mulf %x, %x : {t32}\n"
          f"      %acc = tensor.splat %zero : {tv}\n"
          f"      %ssq = linalg.reduce {{ arith.addf }} ins(%sq : {t32}) outs(%acc : {tv}) dimensions = [1]\n"
          f"      %inv_n_t = tensor.splat %inv_n : {tv}\n"
          f"      %ms = arith.mulf %ssq, %inv_n_t : {tv}\n"
          f"      %eps_t = tensor.splat %eps : {tv}\n"
          f"      %ms_eps = arith.addf %ms, %eps_t : {tv}\n"
          f"      %rstd = math.rsqrt %ms_eps : {tv}\n"
          f"      %bshape = tensor.empty() : {t32}\n"
          f"      %rstd_b = linalg.broadcast ins(%rstd : {tv}) outs(%bshape : {t32}) dimensions = [1]\n"
          f"      %y{'n' if weight else ''} = arith.mulf %x, %rstd_b : {t32}\n"
          + (f"      %y = arith.mulf %yn, %w : {t32}\n" if weight else "") +
          f"      %y16 = arith.truncf %y : {t32} to {t16}\n")
    s += tile("y_tile", "y_view", ["%row", "%c0"], [tile_rows, n_cols], [n_rows, n_cols], "f16", "      ")
    s += tile("r_tile", "rstd_view", ["%row"], [tile_rows], [n_rows], "f32", "      ")
    s += (f"      ktdp.store %y16, %y_tile : {t16}, {at}\n"
          f"      ktdp.store %rstd, %r_tile : {tv}, {atv}\n"
          f"      scf.yield\n    }}\n    return\n  }}\n}}\n")
    return s


def log_softmax_rows(n_rows: int = 64, n_cols: int = 256, cores: int = 4, tile_rows: int = 2) -> str:
    """y = x - max(x) - log(sum(exp(x - max(x)))) per row, f32 arithmetic on f16 data: two reductions
    (maxnumf, addf), the second over an expression of the first, and an output that uses both."""
    R = n_rows // cores
    assert R * cores == n_rows and R % tile_rows == 0
    t16, t32, tv = f"tensor<{tile_rows}x{n_cols}xf16>", f"tensor<{tile_rows}x{n_cols}xf32>", f"tensor<{tile_rows}xf32>"
    at = f"!ktdp.access_tile<{tile_rows}x{n_cols}xindex>"
    s = (f"module {{\n  func.func @log_softmax_kernel(%x_ptr: index, %y_ptr: index) attributes {{grid = [{cores}, 1]}} {{\n"
         f"    %core_id = ktdp.get_compute_tile_id : index\n"
         f"    %c0 = arith.constant 0 : index\n    %step = arith.constant {tile_rows} : index\n"
         f"    %rows = arith.constant {R} : index\n"
         f"    %row0 = arith.muli %core_id, %rows : index\n"
         f"    %row_end = arith.addi %row0, %rows : index\n"
         f"    %zero = arith.constant 0.0 : f32\n"
         f"    %ninf_bits = arith.constant 0xFF800000 : i32\n"
         f"    %ninf = arith.bitcast %ninf_bits : i32 to f32\n")
    s += view("x_view", "x_ptr", [n_rows, n_cols], "f16") + view("y_view", "y_ptr", [n_rows, n_cols], "f16")
    s += "    scf.for %row = %row0 to %row_end step %step {\n"
    s += tile("x_tile", "x_view", ["%row", "%c0"], [tile_rows, n_cols], [n_rows, n_cols], "f16", "      ")
    s += (f"      %x16 = ktdp.load %x_tile : {at} -> {t16}\n"
          f"      %x = arith.extf %x16 : {t16} to {t32}\n"
          f"      %m0 = tensor.splat %ninf : {tv}\n"
          f"      %mx = linalg.reduce {{ arith.maxnumf }} ins(%x : {t32}) outs(%m0 : {tv}) dimensions = [1]\n"
          f"      %bshape = tensor.empty() : {t32}\n"
          f"      %mx_b = linalg.broadcast ins(%mx : {tv}) outs(%bshape : {t32}) dimensions = [1]\n"
          f"      %xc = arith.subf %x, %mx_b : {t32}\n"
          f"      %e = math.exp %xc : {t32}\n"
          f"      %s0 = tensor.splat %zero : {tv}\n"
          f"      %sum = linalg.reduce {{ arith.addf }} ins(%e : {t32}) outs(%s0 : {tv}) dimensions = [1]\n"
          f"      %lse = math.log %sum : {tv}\n"
          f"      %lse_b = linalg.broadcast ins(%lse : {tv}) outs(%bshape : {t32}) dimensions = [1]\n"
          f"      %y = arith.subf %xc, %lse_b : {t32}\n"
          f"      %y16 = arith.truncf %y : {t32} to {t16}\n")
    s += tile("y_tile", "y_view", ["%row", "%c0"], [tile_rows, n_cols], [n_rows, n_cols], "f16", "      ")
    s += f"      ktdp.store %y16, %y_tile : {t16}, {at}\n      scf.yield\n    }}\n    return\n  }}\n}}\n"
    return s


def layernorm_blocked(n_rows: int = 64, n_cols: int = 1024, block: int = 256, cores: int = 4) -> str:
    """Layer norm the way examples/triton-ktir/layernorm_fwd_ktir.mlir writes it (same name, arguments and op
    sequence, sizes of one's choosing): f16 throughout; a row is walked in column blocks of ``block``
    elements — the blocks are summed elementwise into a ``[1, block]`` accumulator carried through an
    ``scf.for``, the accumulator is reduced, mean = sum / N; the same again for the squared deviations;
    rstd = 1 / sqrt(var + eps); mean and rstd are stored per row; a third loop over the blocks writes
    ``(x - mean) * rstd * w + b`` with per-element weights and biases of the input's shape.  Core ``c``
    takes rows ``c, c + cores, ...``."""
    assert n_cols % block == 0
    tb, t1 = f"tensor<1x{block}xf16>", "tensor<1xf16>"
    at, at1 = f"!ktdp.access_tile<1x{block}xindex>", "!ktdp.access_tile<1xindex>"
    s = (f"module {{\n  func.func @_layer_norm_fwd_fused(%X: index, %Y: index, %W: index, %B: index, %Mean: index, "
         f"%Rstd: index, %N: index, %eps: f16, %BLOCK_SIZE: index) attributes {{grid = [{cores}, 1]}} {{\n"
         f"    %core_id = ktdp.get_compute_tile_id : index\n    %c0 = arith.constant 0 : index\n"
         f"    %n_rows = arith.constant {n_rows} : index\n    %n_cores = arith.constant {cores} : index\n"
         f"    %one = arith.constant 1.0 : f16\n")
    for nm in ("X", "Y", "W", "B"):
        s += view(f"{nm}_view", nm, [n_rows, n_cols], "f16")
    s += view("Mean_view", "Mean", [n_rows], "f16") + view("Rstd_view", "Rstd", [n_rows], "f16")
    s += ("    scf.for %row = %core_id to %n_rows step %n_cores : index {\n"
          f"      %zero_block = arith.constant dense<0.0> : {tb}\n"
          f"      %sum_block = scf.for %col = %c0 to %N step %BLOCK_SIZE iter_args(%sum_iter = %zero_block) -> {tb} {{\n")
    s += tile("xa", "X_view", ["%row", "%col"], [1, block], [n_rows, n_cols], "f16", "        ")
    s += (f"        %a = ktdp.load %xa : {at} -> {tb}\n        %sum_next = arith.addf %sum_iter, %a : {tb}\n"
          f"        scf.yield %sum_next : {tb}\n      }}\n"
          f"      %zero_scalar = arith.constant 0.0 : f16\n      %sum_init = tensor.splat %zero_scalar : {t1}\n"
          f"      %reduce_sum = linalg.reduce {{ arith.addf }} ins(%sum_block : {tb}) outs(%sum_init : {t1}) dimensions = [1]\n"
          f"      %N_i32 = arith.index_cast %N : index to i32\n      %N_f16 = arith.sitofp %N_i32 : i32 to f16\n"
          f"      %N_tensor = tensor.splat %N_f16 : {t1}\n      %mean = arith.divf %reduce_sum, %N_tensor : {t1}\n"
          f"      %mean_scalar = tensor.extract %mean[%c0] : {t1}\n      %mean_block = tensor.splat %mean_scalar : {tb}\n"
          f"      %var_block = scf.for %col = %c0 to %N step %BLOCK_SIZE iter_args(%var_iter = %zero_block) -> {tb} {{\n")
    s += tile("xb", "X_view", ["%row", "%col"], [1, block], [n_rows, n_cols], "f16", "        ")
    s += (f"        %a = ktdp.load %xb : {at} -> {tb}\n        %x = arith.subf %a, %mean_block : {tb}\n"
          f"        %x2 = arith.mulf %x, %x : {tb}\n        %var_next = arith.addf %var_iter, %x2 : {tb}\n"
          f"        scf.yield %var_next : {tb}\n      }}\n"
          f"      %var_init = tensor.splat %zero_scalar : {t1}\n"
          f"      %reduce_var = linalg.reduce {{ arith.addf }} ins(%var_block : {tb}) outs(%var_init : {t1}) dimensions = [1]\n"
          f"      %var = arith.divf %reduce_var, %N_tensor : {t1}\n      %eps_tensor = tensor.splat %eps : {t1}\n"
          f"      %var_plus_eps = arith.addf %var, %eps_tensor : {t1}\n      %var_sqrt = math.sqrt %var_plus_eps : {t1}\n"
          f"      %one_tensor = tensor.splat %one : {t1}\n      %rstd = arith.divf %one_tensor, %var_sqrt : {t1}\n"
          f"      %rstd_scalar = tensor.extract %rstd[%c0] : {t1}\n      %rstd_block = tensor.splat %rstd_scalar : {tb}\n")
    s += tile("ma", "Mean_view", ["%row"], [1], [n_rows], "f16", "      ")
    s += tile("ra", "Rstd_view", ["%row"], [1], [n_rows], "f16", "      ")
    s += (f"      ktdp.store %mean, %ma : {t1}, {at1}\n      ktdp.store %rstd, %ra : {t1}, {at1}\n"
          "      scf.for %col = %c0 to %N step %BLOCK_SIZE {\n")
    for nm, vw in (("wa", "W_view"), ("ba", "B_view"), ("xc", "X_view"), ("ya", "Y_view")):
        s += tile(nm, vw, ["%row", "%col"], [1, block], [n_rows, n_cols], "f16", "        ")
    s += (f"        %w = ktdp.load %wa : {at} -> {tb}\n        %b = ktdp.load %ba : {at} -> {tb}\n"
          f"        %xx = ktdp.load %xc : {at} -> {tb}\n        %xm = arith.subf %xx, %mean_block : {tb}\n"
          f"        %xh = arith.mulf %xm, %rstd_block : {tb}\n        %xw = arith.mulf %xh, %w : {tb}\n"
          f"        %y = arith.addf %xw, %b : {tb}\n        ktdp.store %y, %ya : {tb}, {at}\n"
          "        scf.yield\n      }\n      scf.yield\n    }\n    return\n  }\n}\n")
    return s
