#!/usr/bin/env python3
"""Writes the operator inputs of this folder: func @main holding a matmul followed by a row
softmax, in the two spellings the front-end accepts -- the max/exp/sum/div linalg.generic
chain, or one named linalg.softmax -- for the reference's own shape and for the five
benchmark configurations.

    python gen_chains.py            # (re)writes every .mlir file beside this script
"""
import os

HERE = os.path.dirname(os.path.abspath(__file__))


def ttype(dims, elem):
    return "tensor<" + "x".join(str(d) for d in dims) + "x" + elem + ">"


def maps(rank):
    d = ", ".join(f"d{i}" for i in range(rank))
    r = ", ".join(f"d{i}" for i in range(rank - 1))
    return f"affine_map<({d}) -> ({d})>", f"affine_map<({d}) -> ({r})>"


def iters(rank, reduce_last):
    return "[" + ", ".join('"reduction"' if (reduce_last and i == rank - 1) else '"parallel"' for i in range(rank)) + "]"


def chain(batch, M, N, K, in_t="f32", acc_t="f32", out_t="f32", scale=1.0, named=False, title="", arg_t=None):
    """arg_t: element type of the function arguments when it differs from the matmul's operand
    type in_t (f32 arguments rounded to f16 ahead of the matmul)."""
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
    L += [f"    %zero_acc = arith.constant 0.0 : {acc_t}",
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
    if named:
        L += [f"    %sm_empty = tensor.empty() : {c32}",
              f"    %P = linalg.softmax dimension({rank - 1}) ins({cur} : {c32}) outs(%sm_empty : {c32}) -> {c32}"]
    else:
        L += ["    %neg_inf = arith.constant -3.4028235e+38 : f32", "    %zero = arith.constant 0.0 : f32",
              "    // row maximum", f"    %max_empty = tensor.empty() : {red}",
              f"    %max_init = linalg.fill ins(%neg_inf : f32) outs(%max_empty : {red}) -> {red}",
              f"    %max = linalg.generic {{indexing_maps = [{idm}, {drop}], iterator_types = {iters(rank, True)}}}",
              f"        ins({cur} : {c32}) outs(%max_init : {red}) {{",
              "      ^bb0(%in: f32, %acc: f32):", "        %m = arith.maximumf %in, %acc : f32", "        linalg.yield %m : f32", f"      }} -> {red}",
              "    // exp(x - max)", f"    %exp_empty = tensor.empty() : {c32}",
              f"    %exp = linalg.generic {{indexing_maps = [{idm}, {drop}, {idm}], iterator_types = {iters(rank, False)}}}",
              f"        ins({cur}, %max : {c32}, {red}) outs(%exp_empty : {c32}) {{",
              "      ^bb0(%x: f32, %m: f32, %o: f32):", "        %d = arith.subf %x, %m : f32", "        %e = math.exp %d : f32",
              "        linalg.yield %e : f32", f"      }} -> {c32}",
              "    // row sum", f"    %sum_empty = tensor.empty() : {red}",
              f"    %sum_init = linalg.fill ins(%zero : f32) outs(%sum_empty : {red}) -> {red}",
              f"    %sum = linalg.generic {{indexing_maps = [{idm}, {drop}], iterator_types = {iters(rank, True)}}}",
              f"        ins(%exp : {c32}) outs(%sum_init : {red}) {{",
              "      ^bb0(%in: f32, %acc: f32):", "        %s = arith.addf %in, %acc : f32", "        linalg.yield %s : f32", f"      }} -> {red}",
              "    // normalise", f"    %div_empty = tensor.empty() : {c32}",
              f"    %P = linalg.generic {{indexing_maps = [{idm}, {drop}, {idm}], iterator_types = {iters(rank, False)}}}",
              f"        ins(%exp, %sum : {c32}, {red}) outs(%div_empty : {c32}) {{",
              "      ^bb0(%e: f32, %s: f32, %o: f32):", "        %q = arith.divf %e, %s : f32", "        linalg.yield %q : f32", f"      }} -> {c32}"]
    cur = "%P"
    if out_t != "f32":
        elementwise("P16", [f"      ^bb0(%x: f32, %o: {out_t}):", f"        %y = arith.truncf %x : f32 to {out_t}", f"        linalg.yield %y : {out_t}"],
                    [c32], res_t, [cur], "probabilities in the output type")
        cur = "%P16"
    L += [f"    return {cur} : {res_t}", "  }", "}", ""]
    return with_aliases("\n".join(L))


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


def main():
    for name, kw in FILES.items():
        with open(os.path.join(HERE, name), "w") as f:
            f.write(chain(**kw))
        print("wrote", name)


if __name__ == "__main__":
    main()
