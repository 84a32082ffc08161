"""Generates the straight-line CUDA bodies of the channelwise tensor product from the coupling tables.

``python -m fastmace_b200.codegen`` writes ``csrc/generated/tp_generated.cuh`` with, for every node l_max
(0, 1, 2) entering the product:

* ``TpShape<LIN>``: number of paths, input components, components of the scattered message;
* ``tp_forward<LIN>(x, Y, w, acc)``: ``acc[slot] += w[path] * sum_terms coef * x[m_in] * Y[m_edge]``;
* ``tp_backward<LIN, FLIP, NEED_DX>(x, Y, w, wp, g, dY, dr, dx)``: the adjoint of the same expression for one edge and
  one channel given the gradient ``g`` of the receiver's scattered message. ``FLIP`` evaluates the edge in the opposite
  direction (``Y_l -> (-1)^l Y_l``, folded into the coefficients), which is how a receiver-owned walk also produces
  the sender-side gradient of its mirror edge without atomics.

The message layout is K-contiguous for the per-l linear that follows: inside the block of output irrep l the component
index is ``base_l + m * n_seg(l) + seg`` (m the component, seg the path's rank among the paths into l).

All indices are compile-time constants, so ``x``, ``Y``, ``w``, ``acc`` ... live in registers.
"""

from __future__ import annotations

import os

from . import so3

HERE = os.path.dirname(os.path.abspath(__file__))
OUT = os.path.join(HERE, "csrc", "generated", "tp_generated.cuh")


def message_slots(paths):
    """slot[(path, m_out)] -> component index of the K-contiguous message layout; also per-l (base, n_seg)."""
    slots, blocks, base = {}, {}, 0
    for l_out in range(so3.LMAX_SH + 1):
        into = so3.paths_into(paths, l_out)
        blocks[l_out] = (base, len(into))
        for seg, p in enumerate(into):
            for m in range(2 * l_out + 1):
                slots[(p, m)] = base + m * len(into) + seg
        base += len(into) * (2 * l_out + 1)
    return slots, blocks


def _lit(value: float) -> str:
    text = f"{float(value):.9g}"
    if "." not in text and "e" not in text:
        text += ".0"
    return text + "f"


def _emit(lin: int) -> str:
    paths = so3.tp_paths(lin)
    slots, blocks = message_slots(paths)
    in_dim = (lin + 1) ** 2
    mid = so3.mid_dim(paths)
    n_terms = sum(len(p["terms"]) for p in paths)
    out = [f"// ---- node l_max = {lin}: {len(paths)} paths, {mid} message components, {n_terms} coupling terms",
           f"template <> struct TpShape<{lin}> {{",
           f"    static constexpr int kPaths = {len(paths)};",
           f"    static constexpr int kInDim = {in_dim};",
           f"    static constexpr int kMidDim = {mid};",
           "};",
           ""]
    # forward
    out += [f"template <> __device__ __forceinline__ void tp_forward<{lin}>(const float (&x)[{in_dim}], "
            f"const float (&Y)[16], const float (&w)[{len(paths)}], float (&acc)[{mid}]) {{"]
    for p, path in enumerate(paths):
        out.append(f"    // path {p}: {path['l_in']} x {path['l_edge']} -> {path['l_out']}")
        by_out: dict[int, list] = {}
        for mi, me, mo, c in path["terms"]:
            by_out.setdefault(mo, []).append((mi, me, c))
        for mo, terms in sorted(by_out.items()):
            expr = " + ".join(f"{_lit(c)} * x[{path['in_off'] + mi}] * Y[{path['edge_off'] + me}]"
                              for mi, me, c in terms)
            out.append(f"    acc[{slots[(p, mo)]}] = fmaf(w[{p}], {expr}, acc[{slots[(p, mo)]}]);")
    out += ["}", ""]
    # forward, two channels per thread on the packed FP32 pipe (fma.rn.f32x2): the per-channel quantities are pairs,
    # a harmonic times its coupling coefficient is one scalar product shared by the pair
    out += [f"template <> __device__ __forceinline__ void tp_forward_pair<{lin}>(const float2 (&x)[{in_dim}], "
            f"const float (&Y)[16], const float2 (&w)[{len(paths)}], float2 (&acc)[{mid}]) {{"]
    for p, path in enumerate(paths):
        out.append(f"    // path {p}: {path['l_in']} x {path['l_edge']} -> {path['l_out']}")
        by_out = {}
        for mi, me, mo, c in path["terms"]:
            by_out.setdefault(mo, []).append((mi, me, c))
        for mo, terms in sorted(by_out.items()):
            lines = []
            for k, (mi, me, c) in enumerate(terms):
                pair = f"pair_of({_lit(c)} * Y[{path['edge_off'] + me}])"
                xin = f"x[{path['in_off'] + mi}]"
                lines.append(f"float2 e = __fmul2_rn({xin}, {pair});" if k == 0 else f"e = __ffma2_rn({xin}, {pair}, e);")
            slot = slots[(p, mo)]
            out.append(f"    {{ {' '.join(lines)} acc[{slot}] = __ffma2_rn(w[{p}], e, acc[{slot}]); }}")
    out += ["}", ""]
    # backward
    out += [f"template <bool FLIP, bool NEED_DX> __device__ __forceinline__ void tp_backward_{lin}("
            f"const float (&x)[{in_dim}], const float (&Y)[16], const float (&w)[{len(paths)}], "
            f"const float (&wp)[{len(paths)}], const float (&g)[{mid}], float (&dY)[16], float& dr, "
            f"float (&dx)[{in_dim}]) {{"]
    for p, path in enumerate(paths):
        sign = -1.0 if path["l_edge"] % 2 else 1.0
        out.append(f"    {{  // path {p}: {path['l_in']} x {path['l_edge']} -> {path['l_out']}")
        out.append(f"        constexpr float sg = FLIP ? {_lit(sign)} : 1.0f;")
        by_edge: dict[int, list] = {}
        by_in: dict[int, list] = {}
        for mi, me, mo, c in path["terms"]:
            by_edge.setdefault(me, []).append((mi, mo, c))
            by_in.setdefault(mi, []).append((me, mo, c))
        out.append("        float dw = 0.0f;")
        for me, terms in sorted(by_edge.items()):
            expr = " + ".join(f"{_lit(c)} * x[{path['in_off'] + mi}] * g[{slots[(p, mo)]}]" for mi, mo, c in terms)
            ye = path["edge_off"] + me
            out.append(f"        {{ const float s = sg * ({expr}); dw = fmaf(s, Y[{ye}], dw); "
                       f"dY[{ye}] = fmaf(w[{p}], s, dY[{ye}]); }}")
        out.append(f"        dr = fmaf(wp[{p}], dw, dr);")
        out.append("        if (NEED_DX) {")
        for mi, terms in sorted(by_in.items()):
            expr = " + ".join(f"{_lit(c)} * Y[{path['edge_off'] + me}] * g[{slots[(p, mo)]}]" for me, mo, c in terms)
            xi = path["in_off"] + mi
            out.append(f"            dx[{xi}] = fmaf(w[{p}] * sg, {expr}, dx[{xi}]);")
        out.append("        }")
        out.append("    }")
    out += ["}", ""]
    # backward, two channels per thread (packed FP32): x, w, wp, g, dx and the partial sums dY, dr are pairs, the
    # harmonics scalars; a coupling coefficient enters as a constant pair
    out += [f"template <bool FLIP, bool NEED_DX> __device__ __forceinline__ void tp_backward_pair_{lin}("
            f"const float2 (&x)[{in_dim}], const float (&Y)[16], const float2 (&w)[{len(paths)}], "
            f"const float2 (&wp)[{len(paths)}], const float2 (&g)[{mid}], float2 (&dY)[16], float2& dr, "
            f"float2 (&dx)[{in_dim}]) {{"]
    for p, path in enumerate(paths):
        sign = -1.0 if path["l_edge"] % 2 else 1.0
        out.append(f"    {{  // path {p}: {path['l_in']} x {path['l_edge']} -> {path['l_out']}")
        out.append(f"        constexpr float sg = FLIP ? {_lit(sign)} : 1.0f;")
        by_edge = {}
        by_in = {}
        for mi, me, mo, c in path["terms"]:
            by_edge.setdefault(me, []).append((mi, mo, c))
            by_in.setdefault(mi, []).append((me, mo, c))
        out.append("        float2 dw = make_float2(0.0f, 0.0f);")
        for me, terms in sorted(by_edge.items()):
            lines = []
            for k, (mi, mo, c) in enumerate(terms):
                prod = f"__fmul2_rn(x[{path['in_off'] + mi}], g[{slots[(p, mo)]}])"
                coef = f"pair_of(sg * {_lit(c)})"
                lines.append(f"float2 s = __fmul2_rn({prod}, {coef});" if k == 0 else f"s = __ffma2_rn({prod}, {coef}, s);")
            ye = path["edge_off"] + me
            out.append(f"        {{ {' '.join(lines)} dw = __ffma2_rn(s, pair_of(Y[{ye}]), dw); "
                       f"dY[{ye}] = __ffma2_rn(w[{p}], s, dY[{ye}]); }}")
        out.append(f"        dr = __ffma2_rn(wp[{p}], dw, dr);")
        out.append("        if (NEED_DX) {")
        for mi, terms in sorted(by_in.items()):
            lines = []
            for k, (me, mo, c) in enumerate(terms):
                prod = f"__fmul2_rn(g[{slots[(p, mo)]}], pair_of(Y[{path['edge_off'] + me}]))"
                coef = f"pair_of(sg * {_lit(c)})"
                lines.append(f"float2 u = __fmul2_rn({prod}, {coef});" if k == 0 else f"u = __ffma2_rn({prod}, {coef}, u);")
            xi = path["in_off"] + mi
            out.append(f"            {{ {' '.join(lines)} dx[{xi}] = __ffma2_rn(w[{p}], u, dx[{xi}]); }}")
        out.append("        }")
        out.append("    }")
    out += ["}", ""]
    # per-l blocks of the message layout for the host (base component, segments)
    out.append(f"template <> struct TpBlocks<{lin}> {{")
    out.append("    static constexpr int kBase[4] = {" + ", ".join(str(blocks[l][0]) for l in range(4)) + "};")
    out.append("    static constexpr int kSegs[4] = {" + ", ".join(str(blocks[l][1]) for l in range(4)) + "};")
    out.append("};")
    out.append("")
    return "\n".join(out)


def render() -> str:
    head = ["// GENERATED by fastmace_b200/codegen.py from fastmace_b200/so3.py -- do not edit.",
            "// Channelwise (uvu) tensor product of node irreps 0..LIN with spherical harmonics l <= 3 into 0e+1o+2e+3o;",
            "// coefficients are sqrt(2 l_out + 1) * wigner_3j(l_in, l_edge, l_out).",
            "#pragma once",
            "",
            "namespace fmb {",
            "",
            "template <int LIN> struct TpShape;",
            "template <int LIN> struct TpBlocks;",
            "template <int LIN> __device__ __forceinline__ void tp_forward(const float (&x)[(LIN + 1) * (LIN + 1)], "
            "const float (&Y)[16], const float (&w)[LIN == 0 ? 4 : LIN == 1 ? 10 : 17], "
            "float (&acc)[LIN == 0 ? 16 : LIN == 1 ? 40 : 71]);",
            "template <int LIN> __device__ __forceinline__ void tp_forward_pair(const float2 (&x)[(LIN + 1) * (LIN + 1)], "
            "const float (&Y)[16], const float2 (&w)[LIN == 0 ? 4 : LIN == 1 ? 10 : 17], "
            "float2 (&acc)[LIN == 0 ? 16 : LIN == 1 ? 40 : 71]);",
            "__device__ __forceinline__ float2 pair_of(float v) { return make_float2(v, v); }",
            ""]
    body = [_emit(lin) for lin in (0, 1, 2)]
    tail = ["}  // namespace fmb", ""]
    return "\n".join(head + body + tail)


def main() -> str:
    os.makedirs(os.path.dirname(OUT), exist_ok=True)
    text = render()
    old = open(OUT).read() if os.path.exists(OUT) else None
    if old != text:
        with open(OUT, "w") as handle:
            handle.write(text)
    return OUT




# --------------------------------------------------------------------------------------------- symmetric contraction
SYMCON_OUT = os.path.join(HERE, "csrc", "generated", "symcon_generated.cuh")


def _emit_symcon(l_out_max: int) -> str:
    """Straight-line forward and backward of the contraction polynomial for outputs 0..l_out_max.

    ``cf`` points at this thread's coefficient column: term t is ``cf[t * 128]`` (table order = so3.contraction_keys).
    Products of a degree-2 prefix are shared by the degree-3 monomials that extend it, as in the reference's generated
    kernels (fastmace/kernels/cuda/sc_generated.py:65-107)."""
    keys = so3.contraction_keys(l_out_max)
    n_out = (l_out_max + 1) ** 2
    index = {key: t for t, key in enumerate(keys)}
    by_mono: dict[tuple, list] = {}
    for (m_out, nu, mono), t in index.items():
        by_mono.setdefault(mono, []).append((m_out, t))
    deg1 = sorted(m for m in by_mono if len(m) == 1)
    deg2 = sorted(m for m in by_mono if len(m) == 2)
    deg3 = sorted(m for m in by_mono if len(m) == 3)
    prefixes = sorted({m[:2] for m in deg3} | set(deg2))
    fwd = [f"template <> struct SymconShape<{l_out_max}> {{ static constexpr int kTerms = {len(keys)}; "
           f"static constexpr int kOut = {n_out}; }};",
           f"template <> __device__ __forceinline__ void symcon_forward_body<{l_out_max}>(const float (&x)[16], "
           f"const float* __restrict__ cf, float (&y)[{n_out}]) {{"]

    def consume(mono, expr, lines):
        for m_out, t in sorted(by_mono.get(mono, ())):
            lines.append(f"    y[{m_out}] = fmaf(__ldg(cf + {t * 128}), {expr}, y[{m_out}]);")

    for mono in deg1:
        consume(mono, f"x[{mono[0]}]", fwd)
    for pre in prefixes:
        fwd.append(f"    {{ const float p = x[{pre[0]}] * x[{pre[1]}];")
        consume(pre, "p", fwd)
        for mono in (m for m in deg3 if m[:2] == pre):
            consume(mono, f"(p * x[{mono[2]}])", fwd)
        fwd.append("    }")
    fwd += ["}", ""]
    bwd = [f"template <> __device__ __forceinline__ void symcon_backward_body<{l_out_max}>(const float (&x)[16], "
           f"const float* __restrict__ cf, const float (&g)[{n_out}], float (&dx)[16]) {{"]

    def adjoint(mono):
        return " + ".join(f"__ldg(cf + {t * 128}) * g[{m_out}]" for m_out, t in sorted(by_mono[mono]))

    for mono in deg1:
        bwd.append(f"    dx[{mono[0]}] += {adjoint(mono)};")
    for pre in prefixes:
        i, j = pre
        extended = any(m[:2] == pre for m in deg3)
        bwd.append(f"    {{ {f'const float p = x[{i}] * x[{j}]; ' if extended else ''}float hp = 0.0f;")
        if pre in by_mono:
            bwd.append(f"      hp += {adjoint(pre)};")
        for mono in (m for m in deg3 if m[:2] == pre):
            k = mono[2]
            bwd.append(f"      {{ const float h = {adjoint(mono)}; dx[{k}] = fmaf(h, p, dx[{k}]); hp = fmaf(h, x[{k}], hp); }}")
        bwd.append(f"      dx[{i}] = fmaf(hp, x[{j}], dx[{i}]); dx[{j}] = fmaf(hp, x[{i}], dx[{j}]);")
        bwd.append("    }")
    bwd += ["}", ""]
    return "\n".join(fwd + bwd)


def _emit_symcon_group(l_out_max: int) -> str:
    """The same polynomial for R atoms of one species at once: every coefficient is loaded once and used R times
    (the single-atom bodies are bound by their coefficient loads: 410 per atom and channel for outputs 0e + 1o)."""
    keys = so3.contraction_keys(l_out_max)
    n_out = (l_out_max + 1) ** 2
    index = {key: t for t, key in enumerate(keys)}
    by_mono: dict[tuple, list] = {}
    for (m_out, nu, mono), t in index.items():
        by_mono.setdefault(mono, []).append((m_out, t))
    deg1 = sorted(m for m in by_mono if len(m) == 1)
    deg2 = sorted(m for m in by_mono if len(m) == 2)
    deg3 = sorted(m for m in by_mono if len(m) == 3)
    prefixes = sorted({m[:2] for m in deg3} | set(deg2))
    loop = "_Pragma(\"unroll\") for (int r = 0; r < R; ++r)"
    fwd = [f"template <int R> __device__ __forceinline__ void symcon_forward_group_{l_out_max}(const float (&x)[R][16], "
           f"const float* __restrict__ cf, float (&y)[R][{n_out}]) {{"]

    def consume(mono, expr, lines):
        for m_out, t in sorted(by_mono.get(mono, ())):
            lines.append(f"    {{ const float w = __ldg(cf + {t * 128}); {loop} y[r][{m_out}] = fmaf(w, {expr}, y[r][{m_out}]); }}")

    for mono in deg1:
        consume(mono, f"x[r][{mono[0]}]", fwd)
    for pre in prefixes:
        fwd.append(f"    {{ float p[R]; {loop} p[r] = x[r][{pre[0]}] * x[r][{pre[1]}];")
        consume(pre, "p[r]", fwd)
        for mono in (m for m in deg3 if m[:2] == pre):
            consume(mono, f"(p[r] * x[r][{mono[2]}])", fwd)
        fwd.append("    }")
    fwd += ["}", ""]
    bwd = [f"template <int R> __device__ __forceinline__ void symcon_backward_group_{l_out_max}(const float (&x)[R][16], "
           f"const float* __restrict__ cf, const float (&g)[R][{n_out}], float (&dx)[R][16]) {{"]

    def adjoint_into(mono, target, lines):
        for m_out, t in sorted(by_mono[mono]):
            lines.append(f"      {{ const float w = __ldg(cf + {t * 128}); {loop} {target}[r] = fmaf(w, g[r][{m_out}], {target}[r]); }}")

    for mono in deg1:
        bwd.append(f"    {{ float h[R]; {loop} h[r] = 0.0f;")
        adjoint_into(mono, "h", bwd)
        bwd.append(f"      {loop} dx[r][{mono[0]}] += h[r]; }}")
    for pre in prefixes:
        i, j = pre
        bwd.append(f"    {{ float p[R], hp[R]; {loop} {{ p[r] = x[r][{i}] * x[r][{j}]; hp[r] = 0.0f; }}")
        if pre in by_mono:
            adjoint_into(pre, "hp", bwd)
        for mono in (m for m in deg3 if m[:2] == pre):
            k = mono[2]
            bwd.append(f"      {{ float h[R]; {loop} h[r] = 0.0f;")
            adjoint_into(mono, "h", bwd)
            bwd.append(f"        {loop} {{ dx[r][{k}] = fmaf(h[r], p[r], dx[r][{k}]); hp[r] = fmaf(h[r], x[r][{k}], hp[r]); }} }}")
        bwd.append(f"      {loop} {{ dx[r][{i}] = fmaf(hp[r], x[r][{j}], dx[r][{i}]); dx[r][{j}] = fmaf(hp[r], x[r][{i}], dx[r][{j}]); }}")
        bwd.append("    }")
    bwd += ["}", ""]
    return "\n".join(fwd + bwd)


def render_symcon() -> str:
    head = ["// GENERATED by fastmace_b200/codegen.py from fastmace_b200/so3.py -- do not edit.",
            "// Symmetric contraction (correlation 3) of the 16 message components as a polynomial per (atom, channel):",
            "// y[M] = sum_t coef[species][t][channel] * monomial_t(x), terms in the order of so3.contraction_keys.",
            "#pragma once",
            "",
            "namespace fmb {",
            "",
            "template <int LOUT> struct SymconShape;",
            "template <int LOUT> __device__ __forceinline__ void symcon_forward_body(const float (&x)[16], "
            "const float* __restrict__ cf, float (&y)[(LOUT + 1) * (LOUT + 1)]);",
            "template <int LOUT> __device__ __forceinline__ void symcon_backward_body(const float (&x)[16], "
            "const float* __restrict__ cf, const float (&g)[(LOUT + 1) * (LOUT + 1)], float (&dx)[16]);",
            ""]
    return "\n".join(head + [_emit_symcon(l) for l in (0, 1, 2)] + [_emit_symcon_group(l) for l in (0, 1, 2)] +
                     ["}  // namespace fmb", ""])


def _write(path: str, text: str) -> None:
    os.makedirs(os.path.dirname(path), exist_ok=True)
    old = open(path).read() if os.path.exists(path) else None
    if old != text:
        with open(path, "w") as handle:
            handle.write(text)


# --------------------------------------------------------------------------------------------- path-major bodies
PATHS_OUT = os.path.join(HERE, "csrc", "generated", "tp_paths_generated.cuh")


def _emit_paths(lin: int) -> str:
    """One ``TpPath<LIN, P>`` per path: shape constants and the forward of that path alone, for the kernel that takes
    the radial weights of one path at a time from tensor memory."""
    paths = so3.tp_paths(lin)
    slots, blocks = message_slots(paths)
    out = [f"// ---- node l_max = {lin}"]
    seen_in: set[int] = set()
    for p, path in enumerate(paths):
        l_in, l_edge, l_out = path["l_in"], path["l_edge"], path["l_out"]
        n_in, n_e, n_o = 2 * l_in + 1, 2 * l_edge + 1, 2 * l_out + 1
        base, n_seg = blocks[l_out]
        seg = slots[(p, 0)] - base
        first_for_in = l_in not in seen_in
        seen_in.add(l_in)
        out += [f"template <> struct TpPath<{lin}, {p}> {{  // {l_in} x {l_edge} -> {l_out}",
                f"    static constexpr int kNin = {n_in}, kNe = {n_e}, kNo = {n_o};",
                f"    static constexpr int kInOff = {path['in_off']}, kEdgeOff = {path['edge_off']};",
                f"    static constexpr int kSlotBase = {base + seg}, kSlotStride = {n_seg};",
                f"    static constexpr bool kFirstForIn = {'true' if first_for_in else 'false'};",
                f"    static __device__ __forceinline__ void forward(const float (&x)[{n_in}], const float (&Y)[{n_e}], "
                f"float w, float (&acc)[{n_o}]) {{"]
        by_out: dict[int, list] = {}
        for mi, me, mo, c in path["terms"]:
            by_out.setdefault(mo, []).append((mi, me, c))
        for mo, terms in sorted(by_out.items()):
            expr = " + ".join(f"{_lit(c)} * x[{mi}] * Y[{me}]" for mi, me, c in terms)
            out.append(f"        acc[{mo}] = fmaf(w, {expr}, acc[{mo}]);")
        out += ["    }", "};"]
    out.append(f"#define FMB_FOR_EACH_PATH_{lin}(X) " + " ".join(f"X({p})" for p in range(len(paths))))
    out.append("")
    return "\n".join(out)


def render_paths() -> str:
    head = ["// GENERATED by fastmace_b200/codegen.py from fastmace_b200/so3.py -- do not edit.",
            "// The channelwise tensor product one path at a time (same coefficients and message layout as",
            "// tp_generated.cuh): message component of output m is kSlotBase + m * kSlotStride.",
            "#pragma once",
            "",
            "namespace fmb {",
            "",
            "template <int LIN, int P> struct TpPath;",
            ""]
    return "\n".join(head + [_emit_paths(lin) for lin in (1, 2)] + ["}  // namespace fmb", ""])


_tp_main = main


def main() -> str:  # noqa: F811  (both generated headers)
    out = _tp_main()
    _write(SYMCON_OUT, render_symcon())
    _write(PATHS_OUT, render_paths())
    return out


if __name__ == "__main__":
    print(main())
