"""Regenerates the fixtures in this folder from a checkout of the reference project.

Usage:  python tests/golden/make_golden.py /path/to/spn-compiler

What is taken (data files only, no source code):
  * the serialized example models the reference's own tests load (xspn binaries),
  * the stored input / expected-output vectors that accompany NIPS5, nltcs and plants,
    re-packed as compressed .npz (inputs in their narrowest lossless dtype),
  * known_answers.json: the expected values quoted in execute/src/main.cpp:32-52 and the f32
    constants checked by mlir/test/lowering/lospn-to-cpu/lower-to-cpu-nodes-scalar-log.mlir:206-213,340-349.
"""
import json
import os
import shutil
import sys

import numpy as np

HERE = os.path.dirname(os.path.abspath(__file__))


def main(ref):
    ex = os.path.join(ref, "python-interface", "test", "examples")
    models = {
        "NIPS5.bin": os.path.join(ex, "NIPS5", "NIPS5.bin"),
        "nltcs.bin": os.path.join(ex, "nltcs", "nltcs_100_200_2_10_8_8_1_True.bin"),
        "plants.bin": os.path.join(ex, "plants", "plants_100_200_4_3_3_3_1_True.bin"),
        "speaker_FADG0.bin": os.path.join(ex, "speaker", "speaker_FADG0.bin"),
        "NIPS10.bin": os.path.join(ref, "mlir", "test", "test-resources", "NIPS10.bin"),
    }
    for n in ("mini-example", "categorical-example", "gaussian-example", "categorical6", "gaussian10",
              "histogram4"):
        models[n + ".bin"] = os.path.join(ref, "execute", "examples", n + ".bin")
    for dst, src in models.items():
        shutil.copyfile(src, os.path.join(HERE, dst))

    x = np.loadtxt(os.path.join(ex, "NIPS5", "inputdata.txt"), delimiter=";")
    y = np.loadtxt(os.path.join(ex, "NIPS5", "outputdata.txt"))
    assert (x == x.astype(np.uint8)).all()
    np.savez_compressed(os.path.join(HERE, "NIPS5_io.npz"), inputs=x.astype(np.uint8), outputs=y)
    for name, stem in (("nltcs", "nltcs_100_200_2_10_8_8_1_True"), ("plants", "plants_100_200_4_3_3_3_1_True")):
        x = np.loadtxt(os.path.join(ex, name, "input.csv"), delimiter=",")
        y = np.loadtxt(os.path.join(ex, name, stem + "_output.csv"))
        assert (x == x.astype(np.uint8)).all()
        np.savez_compressed(os.path.join(HERE, name + "_io.npz"), inputs=x.astype(np.uint8), outputs=y)

    known = {
        "mini-example": {"dtype": "uint32", "inputs": [[0, 0], [0, 1], [1, 0], [1, 1]],
                         "outputs": [-1.44445, -2.65748, -0.670163, -1.70169]},
        "categorical-example": {"dtype": "uint8", "inputs": [[0, 0], [0, 1], [1, 0], [1, 1]],
                                "outputs": [-2.43612, -1.51983, -1.98413, -1.06784]},
        "gaussian-example": {"dtype": "float32",
                             "inputs": [[0.5, 0.125], [0.125, 0.5], [0.25, 0.25], [0.325, 0.275]],
                             "outputs": [-0.451583, -1.6469, -0.607833, -0.646895]},
        "f32_constants": {
            "categorical_log": {"p": [0.35, 0.55, 0.1], "log": [-1.04982209, -0.597836971, -2.30258512]},
            "gaussian_log": [{"mean": 0.5, "stddev": 1.0, "d": -0.5, "coef": -0.918938517},
                             {"mean": 0.25, "stddev": 0.1, "d": -50.0, "coef": 1.38364661}],
        },
    }
    with open(os.path.join(HERE, "known_answers.json"), "w") as f:
        json.dump(known, f, indent=1)


if __name__ == "__main__":
    if len(sys.argv) != 2:
        sys.exit("usage: make_golden.py <path to a checkout of the reference project>")
    main(sys.argv[1])
