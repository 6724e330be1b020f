from . import hdf5, manifest, native

__all__ = ["hdf5", "manifest", "native"]
