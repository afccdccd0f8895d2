"""Drop-in mirror of the reference's ``omnimem.nsa`` package for the selection path."""
