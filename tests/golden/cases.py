"""Seeded inputs shared by the fixture generator (make_golden.py, which feeds them to
the compiled reference) and by the tests (which feed them to the oracle and to the CUDA
path and compare with the stored reference outputs). numpy's PCG64 stream is stable
across versions, so the inputs are reproducible from the seed alone."""
import numpy as np

X_TRANS = 0
X_NOTRANS = 1
FORM_GENERAL, FORM_BATCHED, FORM_2D = 0, 1, 2


def stored(rng, lead, rows, cols, trans):
    shp = tuple(lead) + ((cols, rows) if trans == X_TRANS else (rows, cols))
    return rng.uniform(-1.0, 1.0, shp).astype(np.float32)


def seeded_cases():
    """(key, form, a, tA, b, tB, alpha, beta, c0) for the reference to run."""
    out = []
    rng = np.random.default_rng(20240)
    ab = [(1.0, 0.0), (0.125, 0.0), (1.0, 1.0), (1.0, 0.5), (-0.75, 0.3)]
    sizes = [(5, 7, 3), (33, 17, 65), (20, 36, 16), (67, 35, 66), (1, 9, 1)]
    n = 0
    for tA in (X_TRANS, X_NOTRANS):
        for tB in (X_TRANS, X_NOTRANS):
            for (alpha, beta) in ab:
                M, N, K = sizes[n % len(sizes)]
                n += 1
                # 2-D
                a = stored(rng, (), M, K, tA)
                b = stored(rng, (), K, N, tB)
                c0 = rng.normal(size=(M, N)).astype(np.float32)
                out.append(("2d", FORM_2D, a, tA, b, tB, alpha, beta, c0))
                # batched, two leading dims
                a = stored(rng, (2, 2), M, K, tA)
                b = stored(rng, (2, 2), K, N, tB)
                c0 = rng.normal(size=(2, 2, M, N)).astype(np.float32)
                out.append(("batched", FORM_BATCHED, a, tA, b, tB, alpha, beta, c0))
                # broadcast: every block of a meets every block of b
                a = stored(rng, (3,), M, K, tA)
                b = stored(rng, (2,), K, N, tB)
                c0 = rng.normal(size=(3, 2, M, N)).astype(np.float32)
                out.append(("broadcast", FORM_GENERAL, a, tA, b, tB, alpha, beta, c0))
                # a.order > 2, b.order == 2 (the flatten shortcut when tA == X_NOTRANS)
                a = stored(rng, (2, 2), M, K, tA)
                b = stored(rng, (), K, N, tB)
                c0 = rng.normal(size=(2, 2, M, N)).astype(np.float32)
                out.append(("a3_b2", FORM_GENERAL, a, tA, b, tB, alpha, beta, c0))
    return out




def mulandshift_cases():
    """(x, w, b, alpha, transposedX, transposedW) for MulAndShift: matrices and a
    higher-order x folded into rows; the transposed forms take matrices only."""
    rng = np.random.default_rng(20241)
    out = []
    for (lead, M, K, N, alpha, tX, tW) in [((), 7, 5, 3, 1.0, X_NOTRANS, X_NOTRANS),
                                           ((2, 3), 16, 24, 40, 1.0, X_NOTRANS, X_NOTRANS),
                                           ((4,), 33, 65, 17, 0.5, X_NOTRANS, X_NOTRANS),
                                           ((), 20, 36, 16, 1.0, X_TRANS, X_NOTRANS),
                                           ((), 67, 35, 66, -0.75, X_NOTRANS, X_TRANS),
                                           ((), 9, 1, 9, 1.0, X_TRANS, X_TRANS)]:
        x = stored(rng, lead, M, K, tX)
        w = stored(rng, (), K, N, tW)
        b = rng.normal(size=(N,)).astype(np.float32)
        out.append((x, w, b, alpha, tX, tW))
    return out


def attention_cases():
    """(q, k, v, mask, scale): small blocks with the head size the fused kernel supports;
    mask None, shared [lenQ, lenK] or per block, with -1e9 entries as padding masks have."""
    rng = np.random.default_rng(20242)
    out = []
    for (blocks, lenQ, lenK, kind) in [(2, 5, 7, "none"), (3, 33, 65, "block"), (2, 130, 200, "shared"),
                                       (1, 1, 1, "none"), (2, 64, 256, "block")]:
        q = rng.normal(size=(blocks, lenQ, 64)).astype(np.float32)
        k = rng.normal(size=(blocks, lenK, 64)).astype(np.float32)
        v = rng.normal(size=(blocks, lenK, 64)).astype(np.float32)
        mask = None
        if kind == "shared":
            mask = np.where(np.arange(lenK)[None, :] > np.arange(lenQ)[:, None] + 70, -1e9, 0.0).astype(np.float32)
        elif kind == "block":
            mask = np.where(rng.uniform(size=(blocks, lenQ, lenK)) < 0.25, -1e9, 0.0).astype(np.float32)
            mask[:, :, 0] = 0.0
        out.append((q, k, v, mask, 0.125))
    return out


def attention_cases_wide():
    """(q, k, v, mask, scale, keep, keep_scale): the transformer sample's default head size of
    128, key sequences beyond one 256-key step, and training-time dropout with a given
    keep-mask (None: inference)."""
    rng = np.random.default_rng(20244)
    out = []
    for (blocks, lenQ, lenK, dim, kind, drop) in [(2, 40, 70, 128, "none", 0.0), (2, 130, 256, 128, "block", 0.0),
                                                  (1, 33, 300, 64, "block", 0.0), (2, 140, 600, 128, "shared", 0.0),
                                                  (2, 50, 90, 64, "none", 0.1), (1, 64, 520, 128, "block", 0.3)]:
        q = rng.normal(size=(blocks, lenQ, dim)).astype(np.float32)
        k = rng.normal(size=(blocks, lenK, dim)).astype(np.float32)
        v = rng.normal(size=(blocks, lenK, dim)).astype(np.float32)
        mask = None
        if kind == "shared":
            mask = np.where(np.arange(lenK)[None, :] > np.arange(lenQ)[:, None] + 300, -1e9, 0.0).astype(np.float32)
        elif kind == "block":
            mask = np.where(rng.uniform(size=(blocks, lenQ, lenK)) < 0.25, -1e9, 0.0).astype(np.float32)
            mask[:, :, 0] = 0.0
        keep, keep_scale = None, 1.0
        if drop > 0:
            keep = (rng.uniform(size=(blocks, lenQ, lenK)) >= drop).astype(np.uint8)
            keep_scale = 1.0 / (1.0 - drop)
        out.append((q, k, v, mask, 1.0 / np.sqrt(dim), keep, keep_scale))
    return out


def output_layer_cases():
    """(h, w): hidden states and a [vocab, hidden] matrix; the third case has logits spread
    wide enough for the -20 floor of the reference's LogSoftmax to act."""
    rng = np.random.default_rng(20243)
    out = []
    for (rows, hidden, vocab, wscale) in [(5, 16, 7, 0.5), (33, 64, 1000, 0.02), (16, 32, 300, 3.0), (3, 8, 1, 1.0)]:
        h = rng.normal(size=(rows, hidden)).astype(np.float32)
        w = (rng.normal(size=(vocab, hidden)) * wscale).astype(np.float32)
        out.append((h, w))
    return out
