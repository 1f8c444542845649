#!/usr/bin/env python3
"""Generator of operator inputs (test infrastructure): func @main holding a matmul followed by a
row softmax, in the two spellings the front-end accepts -- the max/exp/sum/div linalg.generic
chain, or one named linalg.softmax -- plus the two row-only chains of the reference's backend
inputs (row softmax of a given matrix; the layernorm-style variance chain).  The tests build
random and deliberately broken chains with it; run as a script it (re)writes the inputs the
package ships for the reference's own shape and for the five benchmark configurations:

    python tests/chain_gen.py       # writes welder_typical_chain_b200/mlir/*.mlir
"""
import os

HERE = os.path.join(os.path.dirname(os.path.dirname(os.path.abspath(__file__))), "welder_typical_chain_b200", "mlir")


def ttype(dims, elem):
    return "tensor<" + "x".join(str(d) for d in dims) + "x" + elem + ">"


def maps(rank):
    d = ", ".join(f"d{i}" for i in range(rank))
    r = ", ".join(f"d{i}" for i in range(rank - 1))
    return f"affine_map<({d}) -> ({d})>", f"affine_map<({d}) -> ({r})>"


def iters(rank, reduce_last):
    return "[" + ", ".join('"reduction"' if (reduce_last and i == rank - 1) else '"parallel"' for i in range(rank)) + "]"


def softmax_generics(cur, full_t, red_t, rank, result="%P"):
    """The four generics of a row softmax of `cur` (max, exp(x - max), sum, divide); defines `result`."""
    idm, drop = maps(rank)
    return ["    %neg_inf = arith.constant -3.4028235e+38 : f32", "    %zero = arith.constant 0.0 : f32",
            "    // row maximum", f"    %max_empty = tensor.empty() : {red_t}",
            f"    %max_init = linalg.fill ins(%neg_inf : f32) outs(%max_empty : {red_t}) -> {red_t}",
            f"    %max = linalg.generic {{indexing_maps = [{idm}, {drop}], iterator_types = {iters(rank, True)}}}",
            f"        ins({cur} : {full_t}) outs(%max_init : {red_t}) {{",
            "      ^bb0(%in: f32, %acc: f32):", "        %m = arith.maximumf %in, %acc : f32", "        linalg.yield %m : f32", f"      }} -> {red_t}",
            "    // exp(x - max)", f"    %exp_empty = tensor.empty() : {full_t}",
            f"    %exp = linalg.generic {{indexing_maps = [{idm}, {drop}, {idm}], iterator_types = {iters(rank, False)}}}",
            f"        ins({cur}, %max : {full_t}, {red_t}) outs(%exp_empty : {full_t}) {{",
            "      ^bb0(%x: f32, %m: f32, %o: f32):", "        %d = arith.subf %x, %m : f32", "        %e = math.exp %d : f32",
            "        linalg.yield %e : f32", f"      }} -> {full_t}",
            "    // row sum", f"    %sum_empty = tensor.empty() : {red_t}",
            f"    %sum_init = linalg.fill ins(%zero : f32) outs(%sum_empty : {red_t}) -> {red_t}",
            f"    %sum = linalg.generic {{indexing_maps = [{idm}, {drop}], iterator_types = {iters(rank, True)}}}",
            f"        ins(%exp : {full_t}) outs(%sum_init : {red_t}) {{",
            "      ^bb0(%in: f32, %acc: f32):", "        %s = arith.addf %in, %acc : f32", "        linalg.yield %s : f32", f"      }} -> {red_t}",
            "    // normalise", f"    %div_empty = tensor.empty() : {full_t}",
            f"    {result} = linalg.generic {{indexing_maps = [{idm}, {drop}, {idm}], iterator_types = {iters(rank, False)}}}",
            f"        ins(%exp, %sum : {full_t}, {red_t}) outs(%div_empty : {full_t}) {{",
            "      ^bb0(%e: f32, %s: f32, %o: f32):", "        %q = arith.divf %e, %s : f32", "        linalg.yield %q : f32", f"      }} -> {full_t}"]


def row_softmax_chain(M, N, named=False, title="row softmax of a given matrix", aliases=True):
    """X[M,N] f32 -> softmax over each row: the chain without a matmul."""
    full, red = ttype([M, N], "f32"), ttype([M], "f32")
    L = [f"// {title}", "module {", f"  func.func @main(%X: {full}) -> {full} {{"]
    if named:
        L += [f"    %sm_empty = tensor.empty() : {full}", f"    %P = linalg.softmax dimension(1) ins(%X : {full}) outs(%sm_empty : {full}) -> {full}"]
    else:
        L += softmax_generics("%X", full, red, 2)
    L += [f"    return %P : {full}", "  }", "}", ""]
    text = "\n".join(L)
    return with_aliases(text) if aliases else text


def layernorm_variance_chain(M, N, title="row variance, broadcast along the row", aliases=True):
    """A[M,N] f32 -> out[i,j] = (1/N) sum_j (A[i,j] - mean_i)^2 with mean_i = (1/N) sum_j A[i,j]:
    two row reductions, the second depending on the first."""
    full, red = ttype([M, N], "f32"), ttype([M], "f32")
    idm, drop = maps(2)
    id1 = "affine_map<(d0) -> (d0)>"
    inv = repr(1.0 / N)

    def rowsum(name, src):
        return [f"    %{name}_empty = tensor.empty() : {red}",
                f"    %{name}_init = linalg.fill ins(%zero : f32) outs(%{name}_empty : {red}) -> {red}",
                f"    %{name} = linalg.generic {{indexing_maps = [{idm}, {drop}], iterator_types = {iters(2, True)}}}",
                f"        ins({src} : {full}) outs(%{name}_init : {red}) {{",
                "      ^bb0(%in: f32, %acc: f32):", "        %r = arith.addf %in, %acc : f32", "        linalg.yield %r : f32", f"      }} -> {red}"]

    def times_inv(name, src):
        return [f"    %{name}_empty = tensor.empty() : {red}",
                f"    %{name} = linalg.generic {{indexing_maps = [{id1}, {id1}], iterator_types = [\"parallel\"]}}",
                f"        ins({src} : {red}) outs(%{name}_empty : {red}) {{",
                "      ^bb0(%in: f32, %o: f32):", f"        %inv = arith.constant {inv} : f32", "        %v = arith.mulf %in, %inv : f32",
                "        linalg.yield %v : f32", f"      }} -> {red}"]

    L = [f"// {title}", "module {", f"  func.func @main(%A: {full}) -> {full} {{", "    %zero = arith.constant 0.0 : f32"]
    L += ["    // row sum -> mean"] + rowsum("sum", "%A") + times_inv("mean", "%sum")
    L += ["    // (a - mean)^2", f"    %sq_empty = tensor.empty() : {full}",
          f"    %sq = linalg.generic {{indexing_maps = [{idm}, {drop}, {idm}], iterator_types = {iters(2, False)}}}",
          f"        ins(%A, %mean : {full}, {red}) outs(%sq_empty : {full}) {{",
          "      ^bb0(%a: f32, %m: f32, %o: f32):", "        %d = arith.subf %a, %m : f32", "        %s = arith.mulf %d, %d : f32",
          "        linalg.yield %s : f32", f"      }} -> {full}"]
    L += ["    // row sum of the squares -> variance"] + rowsum("sumsq", "%sq") + times_inv("var", "%sumsq")
    L += ["    // broadcast along the row", f"    %out_empty = tensor.empty() : {full}",
          f"    %out = linalg.generic {{indexing_maps = [{drop}, {idm}], iterator_types = {iters(2, False)}}}",
          f"        ins(%var : {red}) outs(%out_empty : {full}) {{",
          "      ^bb0(%v: f32, %o: f32):", "        linalg.yield %v : f32", f"      }} -> {full}",
          f"    return %out : {full}", "  }", "}", ""]
    text = "\n".join(L)
    return with_aliases(text) if aliases else text


def chain(batch, M, N, K, in_t="f32", acc_t="f32", out_t="f32", scale=1.0, named=False, title="", arg_t=None, aliases=True,
          fill="0.0", post_scale=None, extra_add=None):
    """arg_t: element type of the function arguments when it differs from the matmul's operand
    type in_t (f32 arguments rounded to f16 ahead of the matmul).  aliases=False spells every
    type and map in place.  The last three arguments write chains that are NOT the operator (for
    the recogniser's negative tests): a non-zero matmul init, a constant factor applied AFTER
    the division, a constant added to the logits."""
    rank = 3 if batch > 1 else 2
    pre = [batch] if batch > 1 else []
    a_t, b_t = ttype(pre + [M, K], in_t), ttype(pre + [K, N], in_t)
    arg_t = arg_t or in_t
    a_arg, b_arg = ttype(pre + [M, K], arg_t), ttype(pre + [K, N], arg_t)
    c_acc, c32 = ttype(pre + [M, N], acc_t), ttype(pre + [M, N], "f32")
    red = ttype(pre + [M], "f32")
    res_t = ttype(pre + [M, N], out_t)
    idm, drop = maps(rank)
    mm = "linalg.batch_matmul" if batch > 1 else "linalg.matmul"
    L = [f"// {title}", "module {", f"  func.func @main(%A: {a_arg}, %B: {b_arg}) -> {res_t} {{"]
    a_val, b_val = "%A", "%B"
    if arg_t != in_t:
        for nm, src_t, dst_t in (("A", a_arg, a_t), ("B", b_arg, b_t)):
            L += [f"    // {nm} rounded to {in_t} for the matmul", f"    %{nm}n_empty = tensor.empty() : {dst_t}",
                  f"    %{nm}n = linalg.generic {{indexing_maps = [{idm}, {idm}], iterator_types = {iters(rank, False)}}}",
                  f"        ins(%{nm} : {src_t}) outs(%{nm}n_empty : {dst_t}) {{",
                  f"      ^bb0(%x: {arg_t}, %o: {in_t}):", f"        %y = arith.truncf %x : {arg_t} to {in_t}", f"        linalg.yield %y : {in_t}",
                  f"      }} -> {dst_t}"]
        a_val, b_val = "%An", "%Bn"
    L += [f"    %zero_acc = arith.constant {fill} : {acc_t}",
          f"    %c_empty = tensor.empty() : {c_acc}",
          f"    %c_init = linalg.fill ins(%zero_acc : {acc_t}) outs(%c_empty : {c_acc}) -> {c_acc}",
          f"    %C = {mm} ins({a_val}, {b_val} : {a_t}, {b_t}) outs(%c_init : {c_acc}) -> {c_acc}"]
    cur = "%C"

    def elementwise(name, body, in_types, out_type, ins, comment):
        nonlocal L
        n_in = len(ins)
        L += [f"    // {comment}", f"    %{name}_empty = tensor.empty() : {out_type}",
              f"    %{name} = linalg.generic {{indexing_maps = [{', '.join([idm] * (n_in + 1))}], iterator_types = {iters(rank, False)}}}",
              f"        ins({', '.join(ins)} : {', '.join(in_types)}) outs(%{name}_empty : {out_type}) {{"] + body + [f"      }} -> {out_type}"]

    if acc_t != "f32":
        elementwise("C32", [f"      ^bb0(%x: {acc_t}, %o: f32):", f"        %y = arith.extf %x : {acc_t} to f32", "        linalg.yield %y : f32"],
                    [c_acc], c32, [cur], "widen the matmul result before the softmax")
        cur = "%C32"
    if scale != 1.0:
        L.append(f"    %scale = arith.constant {scale!r} : f32")
        elementwise("V", ["      ^bb0(%x: f32, %o: f32):", "        %y = arith.mulf %x, %scale : f32", "        linalg.yield %y : f32"],
                    [c32], c32, [cur], "scaled logits")
        cur = "%V"
    if extra_add is not None:
        L.append(f"    %bias = arith.constant {extra_add!r} : f32")
        elementwise("Vb", ["      ^bb0(%x: f32, %o: f32):", "        %y = arith.addf %x, %bias : f32", "        linalg.yield %y : f32"],
                    [c32], c32, [cur], "a constant added to the logits (not part of the operator)")
        cur = "%Vb"
    if named:
        L += [f"    %sm_empty = tensor.empty() : {c32}",
              f"    %P = linalg.softmax dimension({rank - 1}) ins({cur} : {c32}) outs(%sm_empty : {c32}) -> {c32}"]
    else:
        L += softmax_generics(cur, c32, red, rank)
    cur = "%P"
    if post_scale is not None:
        L.append(f"    %post = arith.constant {post_scale!r} : f32")
        elementwise("Pp", ["      ^bb0(%x: f32, %o: f32):", "        %y = arith.mulf %x, %post : f32", "        linalg.yield %y : f32"],
                    [c32], c32, [cur], "a factor applied after the division (not part of the operator)")
        cur = "%Pp"
    if out_t != "f32":
        elementwise("P16", [f"      ^bb0(%x: f32, %o: {out_t}):", f"        %y = arith.truncf %x : f32 to {out_t}", f"        linalg.yield %y : {out_t}"],
                    [c32], res_t, [cur], "probabilities in the output type")
        cur = "%P16"
    L += [f"    return {cur} : {res_t}", "  }", "}", ""]
    text = "\n".join(L)
    return with_aliases(text) if aliases else text


def with_aliases(text):
    """Names every distinct tensor type and affine map once at the top of the module (`!t0 = ...`,
    `#m0 = ...`), the way MLIR printers do, and uses the names in the body."""
    import re
    title, body = text.split("\n", 1)
    defs = []
    for pattern, sigil in ((r"affine_map<\([^)]*\) -> \([^)]*\)>", "#m"), (r"tensor<[0-9x]+f(?:16|32)>", "!t")):
        seen = []
        for m in re.finditer(pattern, body):
            if m.group(0) not in seen:
                seen.append(m.group(0))
        for i, full in enumerate(seen):
            defs.append(f"{sigil}{i} = {full}")
            body = body.replace(full, f"{sigil}{i}")
    return "\n".join([title] + defs + [body])


FILES = {
    # the reference's own shape, in its three spellings
    "matmul_softmax_chain.mlir": dict(batch=1, M=8192, N=128, K=64, title="decomposed f32 chain at the reference's shape"),
    "matmul_softmax_chain_f16_native.mlir": dict(batch=1, M=8192, N=128, K=64, in_t="f16", acc_t="f16",
                                                 title="f16 operands, f16 matmul result, f32 softmax, f32 result"),
    "matmul_softmax_chain_f16_matmul.mlir": dict(batch=1, M=8192, N=128, K=64, arg_t="f32", in_t="f16", acc_t="f16",
                                                 title="f32 arguments rounded to f16, f16 matmul result, f32 softmax, f32 result"),
    "matmul_softmax_chain_named_softmax.mlir": dict(batch=1, M=8192, N=128, K=64, named=True, title="named linalg.softmax at the reference's shape"),
    # the benchmark configurations
    "cfg1_decomposed_f32_128.mlir": dict(batch=1, M=128, N=128, K=128, title="configuration 1: decomposed f32 chain, 128 cubed"),
    "cfg2_f16_native_4096x1024x1024.mlir": dict(batch=1, M=4096, N=1024, K=1024, in_t="f16", out_t="f16", scale=1.0 / 32,
                                                 title="configuration 2: f16 operands, f32 accumulate, scale 1/32, f16 probabilities"),
    "cfg3_batched_attention_named.mlir": dict(batch=64, M=2048, N=2048, K=128, in_t="f16", out_t="f16", scale=128 ** -0.5, named=True,
                                              title="configuration 3: 64 x (Q[2048,128] . Kt[128,2048]), named softmax, f16 probabilities"),
    "cfg4_vocab_logits.mlir": dict(batch=1, M=8192, N=32000, K=4096, in_t="f16", out_t="f16",
                                   title="configuration 4: hidden[8192,4096] . W[4096,32000], f16 probabilities"),
    "cfg5_skinny_decode.mlir": dict(batch=1, M=16, N=32000, K=4096, in_t="f16", out_t="f16",
                                    title="configuration 5: X[16,4096] . W[4096,32000], f16 probabilities"),
}


# the row-only chains, at the shape of the reference's backend inputs
ROW_FILES = {
    "softmax_row_chain.mlir": lambda: row_softmax_chain(32, 256, title="row softmax of X[32,256] (max -> exp -> sum -> divide), no matmul"),
    "layernorm_variance_chain.mlir": lambda: layernorm_variance_chain(32, 256, title="row variance of A[32,256]: sum -> mean -> squared differences -> sum -> variance -> broadcast"),
}


def main():
    for name, kw in FILES.items():
        with open(os.path.join(HERE, name), "w") as f:
            f.write(chain(**kw))
        print("wrote", name)
    for name, fn in ROW_FILES.items():
        with open(os.path.join(HERE, name), "w") as f:
            f.write(fn())
        print("wrote", name)


if __name__ == "__main__":
    main()
