// Stand-in: nothing from test_utils.h is reached by the oracle.
