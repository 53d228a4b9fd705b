"""Process-wide helpers shared by the package: environment-variable names and the library logger."""
