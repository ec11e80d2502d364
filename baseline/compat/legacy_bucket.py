"""The torch-1.9 ``GradBucket`` surface the reference's hooks were written against.

The reference calls ``bucket.get_tensor()``, ``get_index()``, ``get_per_parameter_tensors()`` and
``is_the_last_bucket_to_allreduce()`` (``communication/powerSGD_hook.py:343,355,386,244``) and
resolves its future to ``[tensor]`` (``:572``).  Today's DDP passes a bucket with ``buffer()``,
``index()``, ``gradients()``, ``is_last()`` and expects the future to resolve to the tensor.
"""
import torch


class LegacyGradBucket:
    __slots__ = ("_b",)

    def __init__(self, bucket):
        self._b = bucket

    def get_tensor(self):
        return self._b.buffer()

    def get_index(self):
        return self._b.index()

    def get_per_parameter_tensors(self):
        return self._b.gradients()

    def is_the_last_bucket_to_allreduce(self):
        return self._b.is_last()

    def __getattr__(self, name):
        return getattr(self._b, name)


def _unwrap(fut):
    value = fut.value()
    return value[0] if isinstance(value, (list, tuple)) else value


def adapt_hook(hook):
    """Wraps a reference hook for ``DistributedDataParallel.register_comm_hook`` of this torch."""

    def adapted(state, bucket):
        return hook(state, LegacyGradBucket(bucket)).then(_unwrap)

    adapted.__name__ = getattr(hook, "__name__", "hook")
    adapted.__qualname__ = getattr(hook, "__qualname__", adapted.__name__)
    return adapted


class HookRegistrar:
    """Stands where the reference's ``get_comm_hooks(args, net, gpu)`` expects the DDP model:
    its only use of ``net`` is ``net.register_comm_hook(state, hook)``
    (``examples/ImageClassification/get_comm_hooks.py:37-122``)."""

    def __init__(self, ddp_model):
        self.ddp_model = ddp_model
        self.state = None
        self.hook = None

    def register_comm_hook(self, state, hook):
        self.state, self.hook = state, hook
        self.ddp_model.register_comm_hook(state, adapt_hook(hook))
