"""Runtime: C-ABI binding, device codec, packed cache, attention backend, generation loop."""
