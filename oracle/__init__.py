"""CPU checkers for the Seera training hot path (test infrastructure only).

`oracle.cpu_oracle` wraps the C restatement (seera_oracle.c); `oracle.ref_engine`
loads the reference's own CPU engine when it has been compiled into oracle/_ref/.
Nothing in the product package imports from here.
"""
