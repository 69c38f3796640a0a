"""spnc: Python front of the SPN compiler, same module layout as the reference's python-interface/spnc."""
