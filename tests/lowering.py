"""Test-side lowering of each PrimDescriptor variant to the (labels_in, labels_out) form the C
oracle takes.  Written independently of the library's own lowering so the two can disagree."""


def lower(desc):
    v = desc.variant
    if v == "BatchedGemm":
        nb = len(desc.batch_dims)
        batch = [100 + i for i in range(nb)]
        return [batch + [0, 2], batch + [2, 1]], batch + [0, 1]
    if v == "Contract":
        return [list(desc.modes_a), list(desc.modes_b)], list(desc.modes_c)
    if v == "ElementwiseMul":
        return None  # rank known only from the operands; handled by the caller
    if v == "Permute":
        return [list(desc.modes_a)], list(desc.modes_b)
    if v == "Reduce":
        return [list(desc.modes_a)], list(desc.modes_c)
    alias = {j: i for i, j in desc.paired}
    if v == "Trace":
        return [[alias.get(m, m) for m in desc.modes_a]], list(desc.modes_c)
    if v in ("AntiTrace", "AntiDiag"):
        return [[alias.get(m, m) for m in desc.modes_a]], [alias.get(m, m) for m in desc.modes_c]
    raise ValueError(v)
