"""Weights in the reference's Keras variable naming.

Each reference layer owns ONE variable, the [fan_in(+1 bias row, last), fan_out] weight, created with
`add_weight(name='fckernel')` (SNN_dense, SNN_TC_Modules.py:57-62) or `name='convkernel'` (SNN_conv,
SNN_TC_Modules.py:134-139). Keras prefixes the layer's own name, which it derives from the class name and the
order of construction: `snn_dense/fckernel:0`, `snn_dense_1/fckernel:0`, `snn_conv/convkernel:0`, ... Those strings
are the keys of the `.npz` files written and read here. The reference's `save_weights('cifar10_best_checkpoint')`
(snntc-cifar10.py:258) writes TensorFlow's own checkpoint format, which needs TensorFlow to read; the bridge is one
line on the reference side:

    np.savez(path, **{v.name: v.numpy() for v in my_model.trainable_variables})      # export
    for v in my_model.trainable_variables: v.assign(npz[v.name])                      # import
"""
import numpy as np
import torch

from .SNN_TC_Modules import SNN_conv, SNN_dense


def keras_names(model):
    """[(variable name, layer)] for the weighted layers of `model` in construction (module) order."""
    out = []
    counts = {"snn_dense": 0, "snn_conv": 0}
    for layer in model.modules():
        if isinstance(layer, SNN_dense):
            base, kernel = "snn_dense", "fckernel"
        elif isinstance(layer, SNN_conv):
            base, kernel = "snn_conv", "convkernel"
        else:
            continue
        n = counts[base]
        counts[base] += 1
        lname = base if n == 0 else "%s_%d" % (base, n)
        out.append(("%s/%s:0" % (lname, kernel), layer))
    return out


def state_in_keras_names(model):
    return {name: layer.weight.detach().cpu().numpy().copy() for name, layer in keras_names(model)}


def save_weights(model, path):
    """Writes `path` (.npz) with one array per layer under its Keras variable name."""
    np.savez(path, **state_in_keras_names(model))


def load_weights(model, path_or_dict, strict=True):
    """Copies the arrays of an .npz file (or a dict) written with Keras variable names into `model`'s layers.
    Shapes must match exactly: [fan_in(+1), fan_out] with the bias row last, conv rows in (kh, kw, c) order."""
    src = path_or_dict if isinstance(path_or_dict, dict) else dict(np.load(path_or_dict))
    used = set()
    for name, layer in keras_names(model):
        if name not in src:
            if strict:
                raise KeyError("no variable %r in the checkpoint (has: %s)" % (name, ", ".join(sorted(src))))
            continue
        arr = np.asarray(src[name], dtype=np.float32)
        if tuple(arr.shape) != tuple(layer.weight.shape):
            raise ValueError("%s: checkpoint shape %s, layer expects %s" % (name, arr.shape, tuple(layer.weight.shape)))
        with torch.no_grad():
            layer.weight.copy_(torch.from_numpy(arr).to(layer.weight.device))
        used.add(name)
    if strict and set(src) - used:
        raise KeyError("checkpoint variables without a layer: %s" % ", ".join(sorted(set(src) - used)))
    return sorted(used)
