"""Hardware probe (nkipy/src/nkipy/runtime/utils.py:3-19 in the reference)."""


def is_device_compatible() -> bool:
    """True when at least one CUDA device is visible to the device runtime."""
    try:
        from ..spike.spike_singleton import visible_device_count

        return visible_device_count() > 0
    except Exception:
        return False


is_neuron_compatible = is_device_compatible
