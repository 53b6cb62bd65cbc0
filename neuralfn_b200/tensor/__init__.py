"""Tensor runtime: stage catalogue, graph compiler, trainers."""
