// Stand-in: METIS is not used by the oracle.
