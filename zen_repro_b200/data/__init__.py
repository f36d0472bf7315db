from .synthetic import ZipfTokenStream, zipf_cdf  # noqa: F401
