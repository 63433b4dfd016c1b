"""CPU checker for the placement-evaluation simulator.

TEST INFRASTRUCTURE ONLY: the parity tests, the smoke test and the
benchmark's CPU-baseline legs use it; the shipped package never imports it.

`oracle.cpu`        ctypes front end of mms_oracle.c (the C restatement)
`oracle.reference`  imports the live reference with import-only stubs, where
                    the reference checkout is present (never on a GPU box)
"""
