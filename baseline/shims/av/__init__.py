"""Stand-in for PyAV (video decoding), which the reference's data utilities import at module load.  The benchmark
feeds synthetic tensors and never opens a video."""
__version__ = "0.0.0+standin"


def open(*a, **k):  # noqa: A001
    raise ImportError("PyAV is not installed on this image (stand-in module)")
