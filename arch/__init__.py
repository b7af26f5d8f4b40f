"""The reference's ``arch`` import root (``from arch.B200 import B200``) over ``deca_b200.arch``."""
