"""Out-of-tree adapters that let the unmodified reference (a byte-identical copy under
``baseline/_ref``) run on the installed PyTorch.  Nothing here is imported by the product
package, and nothing here imports it.

* ``standins/cupy``, ``standins/pynvrtc``: the two call shapes the reference's kernel loader
  uses (``communication/compressors/cupy_kernel.py:1-45``), implemented on the ``cuda-python``
  NVRTC and driver bindings, so that the reference's own CUDA source strings compile and launch
  unchanged.
* ``legacy_bucket``: the torch-1.9 ``GradBucket`` method names the reference's hooks call
  (``communication/powerSGD_hook.py:343,355,386,244``) on top of today's bucket, and a hook
  wrapper that unwraps the ``[tensor]`` the reference's future chain resolves to.
* ``install``: puts ``baseline/_ref`` and the stand-ins on ``sys.path`` and registers the two
  module aliases ``communication/powerSGD_hook.py:8-9`` needs.
"""
