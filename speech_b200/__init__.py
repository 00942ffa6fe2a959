"""speech_b200: a Blackwell-native speech training / inference framework.

Sub-packages: ``core`` (configs, ModelPT, .nemo files, optimizers, trainer), ``ops`` (hand-written sm_100a kernels
with PyTorch reference implementations), ``parallel`` (gradient exchange, sharding, tensor parallelism over
NVLink peer memory), ``modules`` / ``losses`` / ``decoding`` / ``models`` (ASR), ``speechlm``, ``tts``, ``audio``,
``data``, ``tokenizers``, ``inference`` (streaming), ``utils``.
"""
__version__ = "0.1.0"
