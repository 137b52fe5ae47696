"""B200-native batched transformer-policy forward for BeatSaberRL (drop-in for the
reference's ``python/policy.py`` forward path; kernels in ``csrc/``, C ABI in ``include/bsrl.h``)."""

__all__ = ["NotePolicy", "bump_weights_version"]


def __getattr__(name):
    if name in __all__:
        from . import policy
        return getattr(policy, name)
    raise AttributeError(name)
