"""Loads the golden fixtures of tests/golden/ (extracted from gorgonia's own tests)."""
import json
import os

import numpy as np

GOLDEN = os.path.join(os.path.dirname(os.path.abspath(__file__)), "golden")
DT = {"float64": np.float64, "float32": np.float32, "int": np.int64}


def load(name):
    return json.load(open(os.path.join(GOLDEN, name)))


def arr(v):
    """fixture value -> numpy array (0-d for scalars)"""
    a = np.array(v["data"], dtype=DT[v["dtype"]])
    return a.reshape(v["shape"]) if v["kind"] == "tensor" else a.reshape(())


BINOPS = {"Add": "add", "Sub": "sub", "Mul": "mul", "HadamardProd": "mul", "Div": "div", "HadamardDiv": "div"}


def broadcast_div_mod(case):
    """(div, mod, bcast_is_a) of a broadcastAddTests case: which operand is repeated along which
    axis of the 2-D result, in the (i / div) % mod form of b200_binary_bcast."""
    full = case["b"] if case["left"] else case["a"]
    small_is_a = bool(case["left"])
    axis = (case["left"] or case["right"])[0]
    rows, cols = full["shape"]
    # repeated along axis 1: one value per row (index i / cols); along axis 0: one value per column
    return (cols, rows, small_is_a) if axis == 1 else (1, cols, small_is_a)
