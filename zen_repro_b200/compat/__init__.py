"""Reference-shaped API: the same class, method and argument names as the reference's modules, on this
framework's engines.  ``from zen_repro_b200.compat.comm import LoadBalanceAllreduce`` is a drop-in for the
reference's ``from comm import LoadBalanceAllreduce``."""
