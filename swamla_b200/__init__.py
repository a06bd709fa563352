"""B200-native LatentMoE feed-forward path (drop-in for Orolol/swamla's ``LatentMoELayer``).

Host code is PyTorch; the path itself is hand-written CUDA for sm_100a behind a C ABI
(``include/lmoe.h`` -> ``liblmoe.so``).  There is no CPU or library fallback: importing the
operators without the built library raises.
"""
__version__ = "0.1.0"
