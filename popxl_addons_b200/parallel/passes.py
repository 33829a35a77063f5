"""Graph pass: GEMM followed by a tensor-parallel all-reduce becomes one op.

`y = all_reduce(a @ w)` (row-parallel Linear forward, and the data-gradient GEMM of a column-parallel Linear in the
backward pass) is rewritten to `matmul_all_reduce(a, w)`. On one process per GPU that op runs as a single tcgen05 GEMM
kernel whose epilogue pushes every finished tile into all ranks' output buffers with `multimem.red.add` through
NVSwitch, so the reduction overlaps the remaining tiles; elsewhere it runs as matmul + all-reduce.
"""
import torch

from .. import xl
from ..xl.opdef import OPS, OpDef


def _reference_matmul(mm, a, w, native_fn):
    """The torch implementation of a product whose device kernel refused the operands (counted as a fallback)."""
    if native_fn is not None:
        from ..xl.opdef import note_fallback

        note_fallback("matmul", f"{tuple(a.shape)} x {tuple(w.shape)} {a.dtype}")
    return mm.impl(a, w)


def _special_matmul_all_reduce(ex, op, env):
    a, w = env[op.inputs[0]], env[op.inputs[1]]
    native = ex.native_collective("matmul_all_reduce")
    if native is not None:
        res = native(ex, op, a, w)
        if res is not NotImplemented:
            env[op.outputs[0]] = res
            return
    mm = OPS["matmul"]
    fn = mm.native.get(ex.device.type) if ex.use_native else None
    outs = []
    for r in range(ex.num_local):
        y = fn(a[r], w[r]) if fn is not None else NotImplemented
        if y is NotImplemented:
            y = _reference_matmul(mm, a[r], w[r], fn)
        outs.append(y)
    env[op.outputs[0]] = ex.comm.all_reduce(outs, op.attrs["group"], "add", inplace=True)


def _vjp_matmul_all_reduce(ctx, op, gs):
    # forward all-reduce / backward identity, then the ordinary matmul rule
    from ..xl.ops import matmul, reshape, transpose

    (g,) = gs
    a, w = op.inputs
    fa, fw = ctx.fwd(a), ctx.fwd(w)
    ga = matmul(g, transpose(fw))
    gw = matmul(transpose(reshape(fa, (-1, a.shape[-1]))), reshape(g, (-1, g.shape[-1])))
    return [ga, gw]


OpDef("matmul_all_reduce", special=_special_matmul_all_reduce, vjp=_vjp_matmul_all_reduce, collective=True,
      infer=lambda op: [((*op.inputs[0].shape[:-1], op.inputs[1].shape[-1]), op.inputs[0].dtype, ())],
      flops=lambda op: 2 * op.inputs[0].shape[-1] * op.outputs[0].nelms)


def _special_matmul2_all_reduce(ex, op, env):
    a1, w1, a2, w2 = (env[t] for t in op.inputs)
    native = ex.native_collective("matmul2_all_reduce")
    if native is not None:
        res = native(ex, op, a1, w1, a2, w2)
        if res is not NotImplemented:
            env[op.outputs[0]] = res
            return
    mm = OPS["matmul"]
    fn = mm.native.get(ex.device.type) if ex.use_native else None

    def product(a, w):
        y = fn(a, w) if fn is not None else NotImplemented
        return _reference_matmul(mm, a, w, fn) if y is NotImplemented else y

    outs = []
    for r in range(ex.num_local):
        y = product(a1[r], w1[r])
        y += product(a2[r], w2[r])
        outs.append(y)
    env[op.outputs[0]] = ex.comm.all_reduce(outs, op.attrs["group"], "add", inplace=True)


def _vjp_matmul2_all_reduce(ctx, op, gs):
    from ..xl.ops import matmul, reshape, transpose

    (g,) = gs
    grads = []
    g2 = reshape(g, (-1, g.shape[-1]))
    for a, w in ((op.inputs[0], op.inputs[1]), (op.inputs[2], op.inputs[3])):
        fa, fw = ctx.fwd(a), ctx.fwd(w)
        grads += [matmul(g, transpose(fw)), matmul(transpose(reshape(fa, (-1, a.shape[-1]))), g2)]
    return grads


OpDef("matmul2_all_reduce", special=_special_matmul2_all_reduce, vjp=_vjp_matmul2_all_reduce, collective=True,
      infer=lambda op: [((*op.inputs[0].shape[:-1], op.inputs[1].shape[-1]), op.inputs[0].dtype, ())],
      flops=lambda op: 2 * (op.inputs[0].shape[-1] + op.inputs[2].shape[-1]) * op.outputs[0].nelms)


def _matmul_add_ref(c, a, w):
    if c.device.type == "meta":
        return torch.empty_like(c)
    return c + torch.matmul(a, w).to(c.dtype)


def _matmul_add_cuda(c, a, w):
    from ..ops import native

    if c.dim() != 2 or a.dim() != 2 or w.dim() != 2 or not c.is_contiguous():
        return NotImplemented
    res = native.gemm(a, w, out=c, accumulate=1)  # c += a @ w in the GEMM epilogue (c is dead after this op)
    return res


def _vjp_matmul_add(ctx, op, gs):
    from ..xl.ops import matmul, transpose

    (g,) = gs
    c, a, w = op.inputs
    return [g, matmul(g, transpose(ctx.fwd(w))), matmul(transpose(ctx.fwd(a)), g)]


OpDef("matmul_add", impl=_matmul_add_ref, vjp=_vjp_matmul_add,
      flops=lambda op: 2 * op.inputs[1].shape[-1] * op.outputs[0].nelms)
OPS["matmul_add"].native["cuda"] = _matmul_add_cuda


def fuse_matmul_sums(ir: xl.Ir) -> int:
    """`matmul(a1, w1) + matmul(a2, w2)` (both products used by nothing else) -> the second GEMM accumulates into the
    first one's result in its epilogue: one elementwise pass less. Returns the number of rewrites."""
    n = 0
    for g in ir.graphs:
        consumers = {}
        for op in g.ops:
            for t in op.inputs:
                consumers.setdefault(t, []).append(op)
        drop = set()
        for add in g.ops:
            if add.opdef.name != "add" or len(add.inputs) != 2:
                continue
            m1, m2 = add.inputs[0].producer, add.inputs[1].producer
            if any(m is None or m.opdef.name != "matmul" or m.graph is not g or m.uid in drop
                   or len(consumers.get(m.outputs[0], [])) != 1 or m.outputs[0] in g._outputs
                   or m.inputs[0].rank != 2 or m.inputs[1].rank != 2 for m in (m1, m2)):
                continue
            if m1 is m2 or m1.outputs[0].shape != m2.outputs[0].shape or m1.outputs[0].dtype != m2.outputs[0].dtype:
                continue
            # the add becomes `matmul_add(first product, a2, w2)`; the second matmul disappears. Operands of the second
            # product exist before the add, so the op order stays valid.
            add.opdef = OPS["matmul_add"]
            add.name = "matmul_add"
            add.inputs = [m1.outputs[0], m2.inputs[0], m2.inputs[1]]
            add.attrs = {}
            drop.add(m2.uid)
            n += 1
        if drop:
            g.ops = [o for o in g.ops if o.uid not in drop]
    return n


# ---- sequence-parallel forms: GEMM(s) -> reduce-scatter, all-gather -> GEMM ---------------------------------------------


def _special_matmuls_reduce_scatter(ex, op, env):
    vals = [env[t] for t in op.inputs]
    native = ex.native_collective("matmuls_reduce_scatter")
    if native is not None:
        res = native(ex, op, *vals)
        if res is not NotImplemented:
            env[op.outputs[0]] = res
            return
    mm = OPS["matmul"]
    fn = mm.native.get(ex.device.type) if ex.use_native else None

    def product(a, w):
        y = fn(a, w) if fn is not None else NotImplemented
        return _reference_matmul(mm, a, w, fn) if y is NotImplemented else y

    outs = []
    for r in range(ex.num_local):
        y = product(vals[0][r], vals[1][r])
        for i in range(2, len(vals), 2):
            y = y + product(vals[i][r], vals[i + 1][r])
        outs.append(y)
    env[op.outputs[0]] = ex.comm.reduce_scatter(outs, op.attrs["group"], "add")


def _vjp_matmuls_reduce_scatter(ctx, op, gs):
    from ..xl.ops import matmul, reshape, transpose

    a0, w0 = op.inputs[0], op.inputs[1]
    rows, cols = a0.shape[0], w0.shape[-1]
    g = reshape(emit1_all_gather(gs[0], op.attrs["group"]), (rows, cols))
    grads = []
    for i in range(0, len(op.inputs), 2):
        a, w = op.inputs[i], op.inputs[i + 1]
        grads += [matmul(g, transpose(ctx.fwd(w))), matmul(transpose(ctx.fwd(a)), g)]
    return grads


def emit1_all_gather(t, group):
    from ..xl.opdef import emit1

    return emit1("all_gather", [t], dict(group=group))


OpDef("matmuls_reduce_scatter", special=_special_matmuls_reduce_scatter, vjp=_vjp_matmuls_reduce_scatter, collective=True,
      infer=lambda op: [((op.inputs[0].shape[0] * op.inputs[1].shape[-1] // op.attrs["group"].group_size,),
                         op.inputs[0].dtype, ())],
      flops=lambda op: sum(2 * op.inputs[i].shape[-1] * op.inputs[0].shape[0] * op.inputs[1].shape[-1]
                           for i in range(0, len(op.inputs), 2)))


def _special_all_gather_matmul(ex, op, env):
    hs, w = env[op.inputs[0]], env[op.inputs[1]]
    native = ex.native_collective("all_gather_matmul")
    if native is not None:
        res = native(ex, op, hs, w)
        if res is not NotImplemented:
            env[op.outputs[0]], env[op.outputs[1]] = res
            return
    rows, k = op.inputs[0].shape
    full = [f.reshape(rows * op.attrs["group"].group_size, k) for f in ex.comm.all_gather(hs, op.attrs["group"])]
    mm = OPS["matmul"]
    fn = mm.native.get(ex.device.type) if ex.use_native else None
    ys = []
    for r in range(ex.num_local):
        y = fn(full[r], w[r]) if fn is not None else NotImplemented
        ys.append(mm.impl(full[r], w[r]) if y is NotImplemented else y)
    env[op.outputs[0]], env[op.outputs[1]] = ys, full


def _vjp_all_gather_matmul(ctx, op, gs):
    from ..xl.opdef import emit1
    from ..xl.ops import add, matmul, reshape, transpose

    h_s, w = op.inputs
    y, h_full = op.outputs
    gy, gh = gs  # gradient of the product and of the gathered operand (other consumers), either may be None
    parts = []
    if gy is not None:
        parts.append(matmul(gy, transpose(ctx.fwd(w))))
    if gh is not None:
        parts.append(gh)
    g_full = parts[0] if len(parts) == 1 else add(parts[0], parts[1])
    g_s = reshape(emit1("reduce_scatter", [g_full], dict(group=op.attrs["group"], op="add", rts=False)), h_s.shape)
    gw = matmul(transpose(ctx.fwd(h_full)), gy) if gy is not None else None
    return [g_s, gw]


OpDef("all_gather_matmul", special=_special_all_gather_matmul, vjp=_vjp_all_gather_matmul, collective=True,
      infer=lambda op: [((op.inputs[0].shape[0] * op.attrs["group"].group_size, op.inputs[1].shape[-1]),
                         op.inputs[0].dtype, ()),
                        ((op.inputs[0].shape[0] * op.attrs["group"].group_size, op.inputs[0].shape[1]),
                         op.inputs[0].dtype, ())],
      flops=lambda op: 2 * op.inputs[0].shape[1] * op.outputs[0].nelms)


def fuse_sequence_parallel_collectives(ir: xl.Ir) -> int:
    """Rewrites of the sequence-parallel graphs: `reduce_scatter(a1 @ w1 [+ a2 @ w2])` -> `matmuls_reduce_scatter`
    (GEMM epilogues add into the owner's shard) and `reshape(all_gather(h)) @ w` -> `all_gather_matmul` (the first GEMM
    that reads the gathered rows pulls them from the peers itself; its second output, the gathered operand, serves the
    other readers). Returns the number of rewrites."""
    n = 0
    for g in ir.graphs:
        consumers = {}
        for op in g.ops:
            for t in op.inputs:
                consumers.setdefault(t, []).append(op)
        drop = set()

        def single_use_matmul(t):
            m = t.producer
            return (m is not None and m.opdef.name == "matmul" and m.graph is g and m.uid not in drop
                    and len(consumers.get(t, [])) == 1 and t not in g._outputs and m.inputs[0].rank == 2
                    and m.inputs[1].rank == 2)

        for rs in g.ops:
            if rs.opdef.name != "reduce_scatter" or rs.attrs["op"] != "add" or rs.attrs["group"].group_size <= 1:
                continue
            src = rs.inputs[0]
            prod = src.producer
            if prod is None or prod.graph is not g or len(consumers.get(src, [])) != 1 or src in g._outputs:
                continue
            through = []
            if prod.opdef.name == "reshape":  # a view between the sum and the (flattening) reduce-scatter
                through, src = [prod], prod.inputs[0]
                prod = src.producer
                if prod is None or prod.graph is not g or len(consumers.get(src, [])) != 1 or src in g._outputs:
                    continue
            if prod.opdef.name == "matmul" and single_use_matmul(src):
                ins, gone = [prod.inputs[0], prod.inputs[1]], [prod]
            elif prod.opdef.name == "add" and all(single_use_matmul(t) for t in prod.inputs) \
                    and prod.inputs[0].producer is not prod.inputs[1].producer \
                    and prod.inputs[0].shape == prod.inputs[1].shape:
                m1, m2 = prod.inputs[0].producer, prod.inputs[1].producer
                ins, gone = [m1.inputs[0], m1.inputs[1], m2.inputs[0], m2.inputs[1]], [prod, m1, m2]
            else:
                continue
            if ins[0].shape[0] % rs.attrs["group"].group_size:
                continue
            rs.opdef = OPS["matmuls_reduce_scatter"]
            rs.name = "matmuls_reduce_scatter"
            rs.inputs = ins
            rs.attrs = {"group": rs.attrs["group"]}
            drop.update(o.uid for o in gone + through)
            n += 1
        # all_gather -> reshape -> matmul(lhs)
        new_ops = []
        for ag in g.ops:
            if ag.uid in drop:
                continue
            new_ops.append(ag)
            if ag.opdef.name != "all_gather" or ag.attrs["group"].group_size <= 1:
                continue
            h_s, pre = ag.inputs[0], None
            if h_s.rank == 1 and h_s.producer is not None and h_s.producer.opdef.name == "reshape" \
                    and h_s.producer.graph is g and len(consumers.get(h_s, [])) == 1 and h_s not in g._outputs \
                    and h_s.producer.inputs[0].rank == 2:
                pre, h_s = h_s.producer, h_s.producer.inputs[0]  # flattened for the collective: look through the view
            if h_s.rank != 2:
                continue
            users = consumers.get(ag.outputs[0], [])
            if len(users) != 1 or users[0].opdef.name != "reshape" or ag.outputs[0] in g._outputs:
                continue
            rsh = users[0]
            h_full = rsh.outputs[0]
            rows, k = h_s.shape
            if tuple(h_full.shape) != (rows * ag.attrs["group"].group_size, k):
                continue
            mms = [u for u in consumers.get(h_full, []) if u.opdef.name == "matmul" and u.inputs[0] is h_full
                   and u.inputs[1].rank == 2 and u.uid not in drop]
            if not mms:
                continue
            first = min(mms, key=lambda o: g.ops.index(o))
            at = g.ops.index(first)
            if any(g.ops.index(u) < at for u in consumers.get(h_full, []) if u is not first):
                continue  # some other reader of the gathered rows runs before the first product
            # the fused op sits where the first product was; the all-gather and the reshape go away
            first.opdef = OPS["all_gather_matmul"]
            first.name = "all_gather_matmul"
            first.inputs = [h_s, first.inputs[1]]
            first.attrs = {"group": ag.attrs["group"]}
            y = first.outputs[0]
            h_full.producer = first
            first.outputs = [y, h_full]
            drop.update({ag.uid, rsh.uid} | ({pre.uid} if pre is not None else set()))
            new_ops.pop()  # the all_gather just appended
            n += 1
        if drop:
            g.ops = [o for o in g.ops if o.uid not in drop]
    return n


def _fuse_pairs(g) -> int:
    """`all_reduce(matmul(a1, w1) + matmul(a2, w2))` -> one op: both GEMMs push their tiles into the same output."""
    consumers = {}
    for op in g.ops:
        for t in op.inputs:
            consumers.setdefault(t, []).append(op)
    fused, skip = 0, set()
    for ar in g.ops:
        if ar.opdef.name != "all_reduce" or ar.attrs["op"] != "add" or ar.attrs.get("identical_inputs") \
                or ar.attrs["group"].group_size <= 1:
            continue
        add = ar.inputs[0].producer
        if add is None or add.opdef.name != "add" or add.graph is not g or len(consumers.get(add.outputs[0], [])) != 1 \
                or add.outputs[0] in g._outputs:
            continue
        mms = [t.producer for t in add.inputs]
        if any(m is None or m.opdef.name != "matmul" or m.graph is not g or len(consumers.get(m.outputs[0], [])) != 1
               or m.outputs[0] in g._outputs or m.inputs[0].rank != 2 or m.inputs[1].rank != 2 for m in mms):
            continue
        if mms[0] is mms[1] or mms[0].outputs[0].shape != mms[1].outputs[0].shape:
            continue
        # the fused op takes the place of the all-reduce (all four operands exist by then)
        ar.opdef = OPS["matmul2_all_reduce"]
        ar.name = "matmul2_all_reduce"
        ar.inputs = [mms[0].inputs[0], mms[0].inputs[1], mms[1].inputs[0], mms[1].inputs[1]]
        ar.attrs = {"group": ar.attrs["group"]}
        skip.update({add.uid, mms[0].uid, mms[1].uid})
        fused += 1
    if fused:
        g.ops = [o for o in g.ops if o.uid not in skip]
    return fused


def fuse_gemm_collectives(ir: xl.Ir) -> int:
    """Rewrite `matmul -> all_reduce(add)` pairs (matmul result used by nothing else, 2-D weight) and
    `all_reduce(matmul + matmul)` triples in every graph of `ir`. Returns the number of fused collectives. Run after
    autodiff and `apply_pre_alias_patterns`."""
    fused = 0
    for g in ir.graphs:
        fused += _fuse_pairs(g)
    for g in ir.graphs:
        consumers = {}
        for op in g.ops:
            for t in op.inputs:
                consumers.setdefault(t, []).append(op)
        new_ops = []
        skip = set()
        for op in g.ops:
            if op.uid in skip:
                continue
            if op.opdef.name == "matmul" and op.inputs[1].rank == 2 and op.inputs[0].rank == 2:
                y = op.outputs[0]
                users = consumers.get(y, [])
                if (len(users) == 1 and users[0].opdef.name == "all_reduce" and users[0].attrs["op"] == "add"
                        and not users[0].attrs.get("identical_inputs") and y not in g._outputs
                        and users[0].attrs["group"].group_size > 1):
                    ar = users[0]
                    op.opdef = OPS["matmul_all_reduce"]
                    op.name = "matmul_all_reduce"
                    op.attrs = {"group": ar.attrs["group"]}
                    # the fused op produces the all-reduce's output tensor
                    out = ar.outputs[0]
                    out.producer = op
                    op.outputs = [out]
                    skip.add(ar.uid)
                    fused += 1
            new_ops.append(op)
        g.ops = [o for o in new_ops if o.uid not in skip]
    return fused


# ---- overlap: ops that do not need an all-reduce's result move in front of the ops that do ---------------------------------

def _callee_only_updates_operands(callee, _seen=None) -> bool:
    """True if every op of `callee` (and of the graphs it calls) is pure or a plain in-place update of a tensor: such a
    call touches nothing but its own operands. Host streams, remote buffers, collectives and anything else with an
    executor of its own make the call a barrier."""
    seen = _seen if _seen is not None else set()
    if callee in seen:
        return False
    seen.add(callee)
    from ..transforms.recomputation import _is_pure

    for o in callee.ops:
        if _is_pure(o, set()):
            continue
        if o.opdef.name == "call":
            if not _callee_only_updates_operands(o.attrs["graph"], seen):
                return False
            continue
        if o.opdef.inplace and o.opdef.special is None:
            continue
        return False
    return True


def _written_operands(op):
    """Tensors of the op's graph that the op writes: [] for a pure op, None for an op nothing may move across."""
    from ..transforms.recomputation import _is_pure

    if _is_pure(op):
        return []
    name = op.opdef.name
    if name == "call":
        callee = op.attrs["graph"]
        if not _callee_only_updates_operands(callee):
            return None  # host / remote transfers or collectives inside: their order is part of the program
        return [op.inputs[i] for i, t in enumerate(callee._inputs) if callee.is_by_ref(t)]
    if op.opdef.inplace and op.opdef.special is None:
        return [op.inputs[0]]  # the in-place ops of this package update their first operand
    return None


def schedule_collective_overlap(ir: xl.Ir) -> int:
    """Reorder every graph so that an `all_reduce` is followed first by the ops that do not depend on it and only then
    by its consumers. With asynchronous collectives (`comm.async_collectives`) the all-reduce of a tensor-parallel
    block's input gradient then runs under the block's weight-gradient GEMMs. Data dependencies and the order of
    updates to one tensor are kept, so every op computes what it computed before. Returns the number of ops moved."""
    moved = 0
    for g in ir.graphs:
        start = 0
        while True:
            idx = next((i for i in range(start, len(g.ops)) if g.ops[i].opdef.name == "all_reduce"
                        and g.ops[i].attrs["group"].group_size > 1), None)
            if idx is None:
                break
            start = idx + 1
            tainted = set(g.ops[idx].outputs)          # values that exist only after the all-reduce
            read_late, written_late = set(), set()     # operands of the ops that stay behind it
            early, late = [], []
            tail = g.ops[idx + 1:]
            stop = len(tail)
            for j, op in enumerate(tail):
                writes = _written_operands(op)
                if writes is None:
                    stop = j
                    break
                depends = any(t in tainted or t in written_late for t in op.inputs) \
                    or any(t in read_late or t in written_late for t in writes)
                if depends:
                    late.append(op)
                    tainted.update(op.outputs)
                    read_late.update(op.inputs)
                    written_late.update(writes)
                else:
                    if late:
                        moved += 1
                    early.append(op)
            g.ops[idx + 1:] = early + late + tail[stop:]
    return moved
