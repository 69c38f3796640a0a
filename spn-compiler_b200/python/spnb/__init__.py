"""spnb: the B200-native SPN log-likelihood engine's own Python namespace.

  spnb.capi   -- ctypes binding of the C-ABI library (libspnb.so); fails loudly if it is missing
  spnb.synth  -- seeded synthetic SPNs and inputs for the five benchmark configurations
"""
