"""flashrt_b200: the Q2_0 MoE expert path of flashrt, B200-native.

`flashrt_b200.lib` binds the C ABI (libfrx.so); `flashrt_b200.moe` mirrors the reference's
operator interface on torch device tensors; `flashrt_b200.synth` makes the seeded synthetic
weights, activations and router logits the tests and the benchmark use.
"""
__all__ = ["lib", "moe", "synth", "build"]
