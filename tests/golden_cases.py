"""Loader of tests/golden/qlinear_cases.npz (written by tests/golden/make_golden.py)."""
import os

import numpy as np

PATH = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden", "qlinear_cases.npz")


class Case:
    def __init__(self, z, name):
        self.name = name
        self.bits, self.gs, self.O, self.K, self.T, self.sdt, has_bias, self.seed = (int(v) for v in z[name + "_meta"])
        self.q, self.packed = z[name + "_q"], z[name + "_packed"]
        self.scales, self.biases = z[name + "_scales"], z[name + "_biases"]
        self.bias = z[name + "_bias"] if has_bias else None
        self.x, self.y = z[name + "_x"], z[name + "_y"]


def load():
    z = np.load(PATH)
    return [Case(z, str(n)) for n in z["names"]]
