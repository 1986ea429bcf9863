"""torchless_nn_b200: a B200-native (sm_100a) engine for the transformer forward pass of torchless-nn.

The sub-modules carry the reference library's own module names - ``backend``, ``utils``, ``activations``,
``layers``, ``transformer_adapters``, ``network`` - and export the same classes with the same constructor
signatures, so that ``from torchless_nn_b200.network import *`` stands where ``from network import *`` stands in a
user script that runs the reference with ``XP_RUNTIME=B200``.  ``workloads`` holds the benchmark configurations.
Importing the package itself loads nothing; the first import of ``backend`` loads libtlnn.so and fails if it is
missing.
"""
__version__ = "0.1.0"
