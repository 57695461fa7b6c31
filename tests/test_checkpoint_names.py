"""Weights travel under the reference's Keras variable names (SNN_TC_Modules.py:57-62, 134-139)."""
import os
import tempfile

import numpy as np
import pytest


def _model():
    import torch
    from snntc_2023_b200.SNN_TC_Modules import SNN_conv, SNN_dense
    return torch.nn.Sequential(SNN_conv(1, 4, 3, 2), SNN_conv(4, 8, 3, 2), torch.nn.Flatten(),
                               SNN_dense(7 * 7 * 8, 16), SNN_dense(16, 10, biasvolt=0.0))


def test_names_follow_keras_layer_numbering():
    from snntc_2023_b200 import checkpoint
    names = [n for n, _ in checkpoint.keras_names(_model())]
    assert names == ["snn_conv/convkernel:0", "snn_conv_1/convkernel:0", "snn_dense/fckernel:0", "snn_dense_1/fckernel:0"]


def test_round_trip_and_shape_check():
    from snntc_2023_b200 import checkpoint
    a, b = _model(), _model()
    with tempfile.TemporaryDirectory() as d:
        path = os.path.join(d, "w.npz")
        checkpoint.save_weights(a, path)
        z = np.load(path)
        assert z["snn_conv/convkernel:0"].shape == (3 * 3 * 1 + 1, 4)       # bias row last
        assert z["snn_dense_1/fckernel:0"].shape == (16, 10)                # no bias row without bias
        checkpoint.load_weights(b, path)
    for (_, la), (_, lb) in zip(checkpoint.keras_names(a), checkpoint.keras_names(b)):
        assert np.array_equal(la.weight.detach().numpy(), lb.weight.detach().numpy())
    bad = checkpoint.state_in_keras_names(a)
    bad["snn_dense/fckernel:0"] = bad["snn_dense/fckernel:0"][:-1]
    with pytest.raises(ValueError):
        checkpoint.load_weights(b, bad)
    extra = checkpoint.state_in_keras_names(a)
    extra["other/kernel:0"] = np.zeros((1, 1), np.float32)
    with pytest.raises(KeyError):
        checkpoint.load_weights(b, extra)
