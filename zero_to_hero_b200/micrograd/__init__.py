"""Scalar autograd (micrograd): `Value`, `Neuron` / `Layer` / `MLP`, `train`, `to_dot`."""
from .nn import MLP, Layer, Neuron
from .train import train
from .value import BACKEND, Value, live_nodes
from .viz import to_dot

__all__ = ["Value", "Neuron", "Layer", "MLP", "train", "to_dot", "BACKEND", "live_nodes"]
