"""Host seats of the NF4 path: codec, linear and embedding wrappers."""
