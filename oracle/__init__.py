"""CPU checker for the exodus neuron path.  Test infrastructure only: nothing under
``sinabs_exodus_b200`` imports this package."""
