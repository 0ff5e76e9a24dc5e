"""Backend plugin (compiler + driver) in the layout Triton expects of a backend package."""
