"""xspn: the on-disk contract of the SPN engine (Cap'n Proto query files) and the Python objects
that describe a model and a query.  Mirrors the package of the same name in the reference
project (xspn/xspn/**) without depending on SPFlow or pycapnp."""
