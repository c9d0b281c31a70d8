"""Copies the reference's own committed golden vectors for the matmult / linear / conv / unfold2d path
into tests/golden/reference_autograd_data/.

The reference's tests (tests/src/linear_autograd_test.cpp:24-59,128-196, tests/src/conv_autograd_test.cpp:249-374,
tests/src/col_im_autograd_test.cpp:77-116) generate these .npy files with PyTorch and commit them under
tests/autograd_data/; they are data, not source.  Run once in a checkout that has the reference tree:

    python tests/golden/collect_reference_goldens.py <path-to-reference>
"""
import os
import shutil
import sys

NAMES = (
    ["linear_%s.npy" % s for s in ("input", "weight", "bias", "grad", "xgrad", "wgrad", "bgrad")]
    + ["linear_complex_%s.npy" % s for s in ("input_a", "input_b", "weight", "weight2", "bias", "bias2", "grad",
                                             "x1grad", "x2grad", "wgrad", "w2grad", "bgrad", "b2grad")]
    + ["conv2d_%s%s.npy" % (s, e) for s in ("input", "weight", "output", "grad", "xgrad", "wgrad")
       for e in ("", "_batched")]
    + ["unfold_%s.npy" % s for s in ("input", "output", "grad", "input_grad")]
    # grouped conv2d, conv1d and the transposed convolutions (tests/src/conv_autograd_test.cpp:126-240, 284-360, 556-835)
    + ["conv2d_%s%s.npy" % (s, e) for s in ("input", "weight", "output", "grad", "xgrad", "wgrad")
       for e in ("_grouped", "_grouped_batched")]
    + ["%s_%s%s.npy" % (f, s, e) for f in ("conv1d", "conv_transpose1d", "conv_transpose2d")
       for s in ("input", "weight", "output", "grad", "xgrad", "wgrad")
       for e in ("", "_batched", "_grouped", "_grouped_batched")]
    + ["conv_transpose1d_%s_grouped_bigger.npy" % s for s in ("input", "weight", "output", "grad", "xgrad", "wgrad")]
    # conv3d and conv_transpose3d (conv_autograd_test.cpp:376-500, 848-960); the largest sets stay in the reference tree
    + ["conv3d_%s%s.npy" % (s, e) for s in ("input", "weight", "output", "grad", "xgrad", "wgrad")
       for e in ("", "_grouped", "_grouped_batched")]
    + ["conv_transpose3d_%s%s.npy" % (s, e) for s in ("input", "weight", "output", "grad", "xgrad", "wgrad")
       for e in ("", "_grouped_batched")]
)


def main(ref_root):
    src = os.path.join(ref_root, "tests", "autograd_data")
    dst = os.path.join(os.path.dirname(os.path.abspath(__file__)), "reference_autograd_data")
    os.makedirs(dst, exist_ok=True)
    for n in NAMES:
        shutil.copyfile(os.path.join(src, n), os.path.join(dst, n))
    print("copied", len(NAMES), "files to", dst)


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: python tests/golden/collect_reference_goldens.py <path-to-reference>")
    main(sys.argv[1])
