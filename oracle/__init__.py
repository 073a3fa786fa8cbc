"""Test oracle for the sparse-DNN inference path.  TEST INFRASTRUCTURE ONLY: the shipped
package never imports anything from here."""
