"""Parity bookkeeping shared by the GPU tests of the 16-bit tensor-core paths.

Every comparison is put on record in two readings, printed into the test log:
  * max-rel with the error of an element divided by max(|ref|, 1e-2 * rms(ref))  (the Gemm floor)
  * max-rel with the error divided by max(|ref|, rms(ref))                        (the layer floor)
together with the table the reference's own comparison script prints
(examples/data_diff.py:8-25: min / max / mean of the absolute and relative differences and the
number of elements whose absolute difference exceeds 1, 1e-1, ... 1e-7).

Which reading a test asserts on is its own choice and is named in the printed line.  The
attention / layer / stack tests assert on the rms floor: the softmax weights and every tensor
between two kernels are stored in 16 bits, which puts an absolute error of about 2^-11 (fp16)
or 2^-8 (bf16) of the typical magnitude on every output, however small that output is."""
import numpy as np

import oracle


def report(name, ref, got, capsys=None, asserted="rms"):
    """Prints both readings and the data_diff table; returns (max_rel_floor_1e-2rms, max_rel_floor_rms)."""
    ref = np.asarray(ref, dtype=np.float32)
    got = np.asarray(got, dtype=np.float32)
    tight = oracle.max_rel_err(ref, got, floor_frac=1e-2)
    loose = oracle.max_rel_err(ref, got, floor_frac=1.0)
    t = oracle.diff_table(ref, got)
    counts = " ".join(f">{b:g}:{t[f'gt_{b:g}']}" for b in (1, 1e-1, 1e-2, 1e-3, 1e-4, 1e-5, 1e-6, 1e-7))
    line = (f"\n[parity] {name}: {ref.size} elements; max-rel floor 1e-2*rms = {tight:.3e}, floor rms = {loose:.3e} "
            f"(asserted: {asserted}); abs min/max/mean = {t['abs_min']:.3e}/{t['abs_max']:.3e}/{t['abs_mean']:.3e}; "
            f"rel min/max/mean = {t['rel_min']:.3e}/{t['rel_max']:.3e}/{t['rel_mean']:.3e}; abs-diff counts {counts}")
    if capsys is not None:
        with capsys.disabled():
            print(line)
    else:
        print(line)
    return tight, loose
