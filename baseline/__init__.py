"""Runner for the unmodified reference package (installed, git-ignored, under ``baseline/_ref``)."""
