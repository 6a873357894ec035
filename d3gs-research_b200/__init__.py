"""B200-native 3D-Gaussian-splatting training step behind the d3sim.algos.d3gs operator API."""
__version__ = "0.1.0"
