"""Operator layer: CUDA tensors run the sm_100a extension, CPU tensors run the fp32 oracle."""
